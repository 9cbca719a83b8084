/*
 * tritonllm_b200 -- C ABI of the B200 (sm_100a) kernels for the gpt-oss fused
 * per-layer path of TritonLLM.
 *
 * Conventions
 *   - Every pointer named *_dev / every tensor argument is a DEVICE pointer on
 *     the current CUDA device; sizes and strides are in ELEMENTS unless a name
 *     ends in _bytes.  bf16 tensors are passed as void*.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - Every entry point returns an int status: 0 = ok, < 0 = argument rejected
 *     on the host before any launch (B2_ERR_*), > 0 = cudaError_t of the launch.
 *     Nothing throws, synchronises or allocates device memory; scratch is
 *     passed in as a workspace whose size the matching *_workspace_bytes()
 *     function returns.  Launches are asynchronous on `stream` and are safe to
 *     record into a CUDA graph once the library has been used once on the
 *     device (the first call on a device loads the module).
 *   - Device-side waits are bounded; a wait that gives up records a code in a
 *     per-device status word readable with b2_device_status().
 *
 * Each declaration cites the TritonLLM function it stands in for (paths
 * relative to that project's root).
 */
#ifndef TRITONLLM_B200_H
#define TRITONLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_OK 0
#define B2_ERR_NULL (-1)        /* a required pointer is NULL                */
#define B2_ERR_SHAPE (-2)       /* a size is non-positive or inconsistent    */
#define B2_ERR_UNSUPPORTED (-3) /* shape outside what the kernels implement  */
#define B2_ERR_ALIGN (-4)       /* pointer or stride not 16-byte aligned     */
#define B2_ERR_WORKSPACE (-5)   /* workspace missing or too small            */
#define B2_ERR_DRIVER (-6)      /* a driver entry point could not be resolved*/
#define B2_ERR_STATIC_LIMIT (-7) /* larger than the fixed scratch of a *_static entry point */

/* Library ABI version (major*100 + minor). */
int b2_version(void);
/* Human-readable text for a status returned by any entry point. */
const char* b2_status_string(int status);
/* Reads (and with reset != 0 clears) the device status word of the current
 * device; synchronises the device.  0 = no kernel gave up a wait. */
int b2_device_status(int reset, int* status_out);
/* Tuning knobs for experiments ("attn_decode_ctas_per_sm", ...).  Returns
 * B2_ERR_UNSUPPORTED for an unknown name. */
int b2_set_tunable(const char* name, int value);

/* Performance analysis aid: while a device buffer is registered, kernels that support it write
 * 8 int64 values per CTA into it (start and end in nanoseconds, then per-kernel phase stamps or
 * SM-clock totals).  Pass NULL to switch tracing off. */
int b2_set_trace_buffer(void* device_buffer, size_t bytes);

/* Failure-path self-test: launches one small CTA that waits, with the same bounded wait every kernel
 * of the library uses, on an mbarrier nothing will ever arrive on.  The wait gives up after its time
 * limit (about 2 s), the kernel sets the device status word (read it with b2_device_status) and returns;
 * the context stays usable.  No counterpart in the reference. */
int b2_selftest_wait_timeout(void* stream);

/* ---- RMSNorm ---------------------------------------------------------------
 * y = x * rsqrt(sum(x^2)/dim + eps) * gain, rows of `dim` bf16, gain fp32.
 * Replaces rmsnorm_forward / rmsnorm_kernel
 * (tritonllm/gpt_oss/triton/triton_kernels.py:9-35; callers model.py:68,476,754,923).
 * `out` may alias `x`.  dim % 8 == 0, dim <= 8192. */
int b2_rmsnorm(const void* x, const float* gain, void* out, int64_t rows, int dim, float eps, void* stream);

/* h = bf16(x + delta); y = rmsnorm(h).  Fuses the residual adds
 * `t = x + t` (model.py:572) / `x.add_(t)` (model.py:816) into the following
 * RMSNorm (model.py:476,754).  h_out may alias x or delta; y_out must not. */
int b2_add_rmsnorm(const void* x, const void* delta, const float* gain, void* h_out, void* y_out, int64_t rows,
                   int dim, float eps, void* stream);

/* ---- RoPE ------------------------------------------------------------------
 * In-place half-split rotary on q [B,T,Hq,D] and k [B,T,Hkv,D] (contiguous
 * bf16), position (t + *offset_dev) % max_ctx, tables fp32 [max_ctx, D/2].
 * Replaces rope_forward / rope_kernel (triton_kernels.py:38-108). D == 64. */
int b2_rope_inplace(void* q, void* k, const float* sin_tab, const float* cos_tab, const int64_t* offset_dev,
                    int64_t batch, int64_t tokens, int n_q_heads, int n_kv_heads, int head_dim, int64_t max_ctx,
                    void* stream);

/* ---- decode: QKV + bias + RoPE + KV-cache write ------------------------------
 * One new token per sequence: qkv = hidden[b] @ W^T + bias (fp32 accumulate),
 * q and k heads rotated at position *offset_dev % max_ctx, q -> q_out
 * [B, Hq*D] bf16, k/v -> cache_{k,v}[b, *offset_dev, head, :].
 * Replaces qkv_rope_cache_decode_forward and its split-K + reduce kernels
 * (triton_kernels.py:865-1255; caller model.py:489-503).
 * W [(Hq+2Hkv)*D, hidden] bf16 row-major, hidden % 64 == 0, D == 64.
 * cache strides in elements: batch, position, head (innermost stride 1);
 * cache_ctx = positions per sequence.  An offset outside [0, cache_ctx) writes
 * no K/V and records B2_DEV_BAD_INDEX in the device status word. */
int b2_qkv_rope_kv_decode(const void* hidden, int64_t hidden_stride_b, const void* weight, const void* bias,
                          const float* sin_tab, const float* cos_tab, const int64_t* offset_dev, void* q_out,
                          void* cache_k, void* cache_v, int64_t cache_stride_b, int64_t cache_stride_n,
                          int64_t cache_stride_h, int64_t cache_ctx, int64_t batch, int hidden_size, int n_q_heads,
                          int n_kv_heads, int head_dim, int64_t max_ctx, void* stream);

/* The same with one position per sequence and, optionally, a paged KV store - what a batched server needs
 * (the reference keeps ONE position for the whole batch, model.py:344, 487, so it has no counterpart of this
 * form; the arithmetic is that of qkv_rope_cache_decode_forward, triton_kernels.py:1109-1255).
 * positions_dev: int64 [batch]; sequence b's q and k are rotated at positions_dev[b] % max_ctx and its K/V row
 * goes to token positions_dev[b] of its own store.  block_table == NULL: kv_k / kv_v are [batch, kv_ctx, heads, 64]
 * at the given strides.  block_table int32 [batch, table_stride] (page_size > 0): kv_k / kv_v are a pool of pages
 * [pages, page_size, heads, 64], kv_stride_b is the page stride, and token p of sequence b lives in page
 * block_table[b][p / page_size], row p % page_size; kv_ctx (<= table_stride * page_size) is the capacity of a
 * sequence.  A position outside [0, kv_ctx) or an unmapped (negative) page writes no K/V and records
 * B2_DEV_BAD_INDEX. */
int b2_qkv_rope_kv_decode_ragged(const void* hidden, int64_t hidden_stride_b, const void* weight, const void* bias,
                                 const float* sin_tab, const float* cos_tab, const int64_t* positions_dev, void* q_out,
                                 void* kv_k, void* kv_v, int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h,
                                 int64_t kv_ctx, const int32_t* block_table, int64_t table_stride, int page_size,
                                 int64_t batch, int hidden_size, int n_q_heads, int n_kv_heads, int head_dim,
                                 int64_t max_ctx, void* stream);

/* ---- decode: o_proj + bias + residual, written into the residual -------------
 * residual[b,:] = t[b,:] @ W^T + bias + residual[b,:]   (one rounding to bf16).
 * Replaces out_residual_decode_forward / out_residual_decode_kernel
 * (triton_kernels.py:1258-1346,1470-1517; caller model.py:199-215,567-569).
 * W [n_out, k_in] bf16 row-major, k_in % 64 == 0. */
int b2_oproj_residual_decode(const void* t, int64_t t_stride_b, const void* weight, const void* bias, void* residual,
                             int64_t residual_stride_b, int64_t batch, int k_in, int n_out, void* stream);

/* ---- prefill projections on the tensor cores (tcgen05 / TMEM) --------------------
 * All three compute  A[M,K] (bf16, row stride ld) times W[N,K]^T (bf16 row-major, the
 * layout the model stores) with fp32 accumulation.  K % 8 == 0, ld % 8 == 0.
 *
 * b2_linear_bias: out = x W^T + bias (bf16).  Replaces QKV.forward / OUT.forward
 * (tritonllm/gpt_oss/triton/model.py:136-138, 195-197). */
int b2_linear_bias(const void* x, int64_t ldx, const void* weight, const void* bias, void* out, int64_t ld_out,
                   int64_t M, int N, int K, void* stream);

/* QKV projection with the bias, the split into heads and the YaRN RoPE fused into the
 * epilogue: row m = b*tokens + t is rotated at position (t + *offset_dev) % max_ctx;
 * q -> q_out [B,T,Hq,64]; k and v -> k_out / v_out at [b, t (+ *offset_dev when
 * kv_add_offset != 0), head, :] with the element strides given (fresh [B,T,Hkv,64]
 * tensors, or the KV cache itself; rows outside [0, kv_ctx) are not written).
 * round_before_rope != 0 rounds the projection to bf16 before rotating, as the
 * reference's unfused path does.  Replaces QKV.forward + torch.split + 3x contiguous +
 * rope_forward + Cache.extend (model.py:506-526, triton_kernels.py:38-108, model.py:426-433). */
int b2_qkv_rope_prefill(const void* x, int64_t ldx, const void* weight, const void* bias, const float* sin_tab,
                        const float* cos_tab, const int64_t* offset_dev, void* q_out, void* k_out, void* v_out,
                        int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, int64_t kv_ctx,
                        int kv_add_offset, int64_t batch, int64_t tokens, int hidden_size, int n_q_heads,
                        int n_kv_heads, int head_dim, int64_t max_ctx, int round_before_rope, void* stream);

/* out = t W^T + bias + residual, one rounding to bf16; out may alias residual.
 * Replaces OUT.forward followed by `t = x + t` (model.py:571-572). */
int b2_oproj_residual(const void* t, int64_t ldt, const void* weight, const void* bias, const void* residual,
                      int64_t ld_res, void* out, int64_t ld_out, int64_t M, int N, int K, void* stream);

/* Router logits: logits = bf16_round(x Wg) + bias, fp32 [M, n_experts].  The gate weight is
 * passed expert-major, [n_experts, K] (the transpose of the [K, n_experts] tensor the
 * reference keeps, model.py:592-598,991-994); gate_bias fp32 may be NULL.
 * Replaces torch.matmul(x, wg).float() + bg (tritonllm/gpt_oss/triton/moe.py:46-48,108-110). */
int b2_router_logits(const void* x, int64_t ldx, const void* gate_weight_ek, const float* gate_bias, float* logits,
                     int64_t ld_logits, int64_t M, int n_experts, int K, void* stream);

/* ---- prefill attention (tcgen05 / TMEM) --------------------------------------------
 * Causal GQA attention with per-head sinks and an optional sliding window for `tokens`
 * query tokens at absolute positions *start_q_dev .. +tokens-1: key j is visible to the
 * query at position p iff j <= p, j < n_kv_ctx and (window == 0 or j >= p - window + 1).
 * q [B, T, Hkv*G, 64] bf16 contiguous (head h = kv*G + g), k/v bf16 [B, n_kv_ctx, Hkv, 64]
 * with element strides (batch, position, head) - the native layout of the projections
 * and of the KV cache, no transposed copies -, out [B, T, Hkv*G*64] bf16.
 * Replaces attention / _attn_fwd (tritonllm/gpt_oss/triton/attention_tt_tma.py:17-163,
 * attention_tt.py; caller model.py:556-565) and attention_ref for short prompts
 * (attention_ref.py:4-42, model.py:546-555).  Rows of k/v at positions a query block can
 * load but not see must hold finite values (a zero-initialised cache does). D == 64. */
int b2_attn_prefill(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                    int64_t batch, int64_t tokens, int64_t n_kv_ctx, int n_kv_heads, int group, int head_dim,
                    int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window,
                    const void* start_q_dev, int start_q_is_i64, void* stream);

/* ---- decode attention --------------------------------------------------------
 * One query token per sequence at absolute position *start_q_dev against a
 * contiguous KV cache: keys [lo,hi), hi = min(start_q+1, n_kv_ctx),
 * lo = window ? max(0, start_q-window+1) : 0; per-head sink logit joins the
 * softmax denominator.  Replaces attention_decode and its single / split-K /
 * reduce kernels (tritonllm/gpt_oss/triton/attention_tt_decode.py:9-408;
 * caller model.py:536-545).
 * q [B, Hkv*G*D] bf16 (head h = kv*G + g), k/v bf16 with element strides
 * (batch, position, head), out [B, Hkv*G*D] bf16.  sinks: bf16 or fp32 [Hkv*G]
 * (may be NULL = 0).  start_q_dev: int32 or int64 scalar on the device.
 * D == 64, G <= 8.  The workspace must be zero-filled once after allocation;
 * the kernel leaves it reusable by the next call on the same stream. */
size_t b2_attn_decode_workspace_bytes(int64_t batch, int n_kv_heads, int group);
int b2_attn_decode(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                   int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx, int64_t kv_stride_b,
                   int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window, const void* start_q_dev,
                   int start_q_is_i64, void* workspace, size_t workspace_bytes, void* stream);

/* Decode attention with one position per sequence and, optionally, a paged KV store (same role as
 * b2_qkv_rope_kv_decode_ragged; the arithmetic is that of attention_decode, attention_tt_decode.py:291-408).
 * positions_dev: int32 or int64 [batch]; sequence b sees keys [lo_b, hi_b) computed from its own position.
 * block_table == NULL: k / v as in b2_attn_decode.  Otherwise k / v are a pool [n_pages, page_size, heads, 64]
 * (kv_stride_b = page stride), block_table int32 [batch, table_stride], page_size a multiple of 32, and n_kv_ctx
 * (<= table_stride * page_size) the capacity of a sequence; an unmapped (negative) page that the visible range
 * reaches records B2_DEV_BAD_INDEX.  batch <= 2048.  Workspace as for b2_attn_decode (same size function). */
int b2_attn_decode_ragged(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                          int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx, int64_t kv_stride_b,
                          int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window, const void* positions_dev,
                          int positions_are_i64, const int32_t* block_table, int64_t table_stride, int page_size,
                          int64_t n_pages, void* workspace, size_t workspace_bytes, void* stream);

/* Decode attention for callers that cannot allocate device memory (a process whose
 * memory is carved up in advance, a plugin under a runtime that owns the allocator):
 * same arguments and results as b2_attn_decode, minus the workspace.  The split-KV
 * partials and counters live in a fixed ~5.4 MiB array inside the library image, so
 * every GPU that loads the library holds that memory until exit, and the problem is
 * bounded: batch * n_kv_heads <= b2_attn_decode_static_max_units() (4096)
 * and at most 160 SMs, otherwise B2_ERR_STATIC_LIMIT.  It calls no cudaMalloc/cudaFree or other allocating routine.
 * The first call on a device looks up the array's device address; make that call
 * before any stream capture begins.  All calls on a device share the array (the
 * counters are cleared on `stream` before each launch): calls that can overlap on
 * the GPU race on it and must be serialised by the caller.
 * This entry point has no counterpart in the reference. */
size_t b2_attn_decode_static_max_units(void);
int b2_attn_decode_static(const void* q, const void* k, const void* v, const void* sinks, int sinks_is_f32, void* out,
                          int64_t batch, int n_kv_heads, int group, int head_dim, int64_t n_kv_ctx,
                          int64_t kv_stride_b, int64_t kv_stride_n, int64_t kv_stride_h, float sm_scale, int window,
                          const void* start_q_dev, int start_q_is_i64, void* stream);

/* ---- clamped SwiGLU ------------------------------------------------------------
 * a [rows, 2n] bf16 with gate = even / linear = odd columns -> out [rows, n]:
 * g = min(g,limit); l = clamp(l,-limit,limit); s = g/(1+exp(-alpha g)); out = s*l+s.
 * limit <= 0 disables clamping.  Replaces swiglu / _swiglu
 * (tritonllm/triton_kernels/swiglu.py:25-86, swiglu_details/_swiglu.py:37-102)
 * and moe.swiglu (tritonllm/gpt_oss/triton/moe.py:25-33). */
int b2_swiglu(const void* a, int64_t a_stride_row, void* out, int64_t out_stride_row, int64_t rows, int64_t n,
              float alpha, float limit, void* stream);

/* ---- router top-k + softmax ------------------------------------------------------
 * Per row of fp32 logits [rows, n_experts]: the k largest by (IEEE-bits key
 * descending, expert index ascending), emitted sorted by expert id ascending;
 * vals = softmax over the k winners (fp32) or the raw logits; idx int16;
 * bitmatrix uint32 word (row, e/32) bit e%32 at element strides (bm_stride_row,
 * bm_stride_word); `zero_scratch` (may be NULL) int32[zero_scratch_len] is
 * cleared.  Replaces topk / _topk_forward
 * (tritonllm/triton_kernels/topk.py:8-53, topk_details/_topk_forward.py:38-146).
 * k <= 8, n_experts <= 1024. */
int b2_topk_softmax(const float* logits, int64_t logits_stride_row, int64_t rows, int n_experts, int k,
                    int apply_softmax, float* vals, int16_t* idx, uint32_t* bitmatrix, int64_t bm_stride_row,
                    int64_t bm_stride_word, int32_t* zero_scratch, int zero_scratch_len, void* stream);

/* ---- MXFP4 -> bf16 ------------------------------------------------------------------
 * out[r, k] = E2M1(codes[r, k/2] nibble k%2) * 2^(scales[r, k/32] - 127), rounded to bf16.
 * codes uint8 [rows, k/2] (low nibble = even k), scales uint8 E8M0 [rows, k/32], k % 32 == 0,
 * all contiguous along k.  Same arithmetic as upcast_from_mxfp_torch
 * (tritonllm/triton_kernels/numerics_details/mxfp.py:237-299) and the checkpoint decoder
 * (tritonllm/gpt_oss/triton/weights.py:68-117). */
int b2_mxfp4_upcast(const void* codes, const void* scales, void* out, int64_t rows, int64_t k, void* stream);

/* ---- MoE expert MLP, decode-sized batches ---------------------------------------------
 * For every routed (token t, slot k) with expert e = topk_idx[t,k] and weight g = topk_w[t,k]:
 *   a = swiglu(x[t] W1[e] + b1[e])        W1[e]: [hidden] -> [2*intermediate], columns interleaved
 *                                          (even = gate, odd = linear), a is a bf16 tensor
 *   y = (a W2[e] + b2[e]) * g             bf16 tensor
 * out[t] = sum_k y (fp32, slot order), bf16.  Replaces moe_decode_experts / moe_experts
 * (tritonllm/gpt_oss/triton/moe.py:54-87,118-175) = matmul_ogs with gather + fused SwiGLU, then
 * matmul_ogs with scatter and gammas (tritonllm/triton_kernels/matmul_ogs.py:376-593; torch twin
 * :600-665), driven by the routing data of routing() (tritonllm/triton_kernels/routing.py:292-303).
 * Weights are MXFP4 as the reference stores them in memory, K contiguous: codes uint8
 * [E, N, K/2] (low nibble = even k), with the E8M0 scales as [E, N, K/32] (the reference keeps
 * them [E, K/32, N]: transpose once at load).  Biases fp32 [E, N] (the reference's fp32 bias
 * caches).  topk_idx int16 [tokens, 4] / topk_w fp32 [tokens, 4] as b2_topk_softmax writes them.
 * tokens <= 256, n_experts <= 128, hidden and intermediate multiples of 64; scale bytes 1..254.
 * workspace: 256-byte aligned device memory of b2_moe_decode_workspace_bytes(); it need not be
 * zeroed.  Experts that received no token are not read. */
size_t b2_moe_decode_workspace_bytes(int64_t tokens, int hidden, int intermediate);
int b2_moe_experts_decode(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w,
                          const void* w1_codes, const void* w1_scales, const float* b1, const void* w2_codes,
                          const void* w2_scales, const float* b2, void* out, int64_t ld_out, void* workspace,
                          size_t workspace_bytes, int64_t tokens, int n_experts, int hidden, int intermediate,
                          float alpha, float limit, void* stream);

/* The same operation on the tensor cores' block-scaled FP4 path (tcgen05.mma.kind::mxf8f6f4): the codes
 * and their scales are consumed as they are, activations are split into two block-scaled E4M3 terms
 * (exact for bf16 inputs).  Weight layout: codes uint8 [E, N, Kp/2] with Kp = K rounded up to 128 and the
 * padding zero, 32-byte aligned; scales as 512-byte blocks [E, ceil(N/128), Kp/128, 32, 4, 4]:
 * block (e, t, b) byte [i][j][k] = scale of row 128 t + 32 j + i for K elements 128 b + 32 k .. + 31
 * (127 where the row or the group does not exist).  tokens <= 2048 (an expert's tokens are spread over
 * CTAs of 32 or 64); everything else as b2_moe_experts_decode. */
size_t b2_moe_fp4_workspace_bytes(int64_t tokens, int hidden, int intermediate);
int b2_moe_experts_decode_fp4(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w,
                              const void* w1_codes, const void* w1_sf, const float* b1, const void* w2_codes,
                              const void* w2_sf, const float* b2, void* out, int64_t ld_out, void* workspace,
                              size_t workspace_bytes, int64_t tokens, int n_experts, int hidden, int intermediate,
                              float alpha, float limit, void* stream);

/* With out == NULL b2_moe_experts_decode_fp4 stops before the sum over a token's experts and leaves the expert
 * outputs in the workspace; b2_moe_combine_add_rmsnorm then does that sum together with what the model does
 * next (x.add_(t) of MLPBlock.forward, tritonllm/gpt_oss/triton/model.py:816, and the norm that follows,
 * model.py:476 or :923): delta[t] = bf16(sum_k y), h_out = bf16(residual + delta), y_out = RMSNorm(h_out) * gain.
 * workspace, tokens, hidden, intermediate: those of the b2_moe_experts_decode_fp4 call before it on the stream.
 * residual, h_out, y_out [tokens, hidden] bf16 (row strides in elements, multiples of 8; h_out may be residual),
 * gain fp32 [hidden]; hidden <= 3072. */
int b2_moe_combine_add_rmsnorm(const void* workspace, size_t workspace_bytes, int64_t tokens, int hidden,
                               int intermediate, const void* residual, int64_t residual_stride, const float* gain,
                               float eps, void* h_out, int64_t h_stride, void* y_out, int64_t y_stride, void* stream);

/* ---- MoE expert MLP, prompt-sized batches ------------------------------------
 * The same computation as b2_moe_experts_decode_fp4 for thousands of tokens at once: the tokens routed to an
 * expert are the M rows of a grouped GEMM (256-row tiles on CTA pairs, tcgen05, bf16), so the work is tensor-bound
 * instead of re-streaming every weight tile per 32 tokens.  Replaces moe_experts (gpt_oss/triton/moe.py:54-87):
 * routing metadata (triton_kernels/routing.py:93-166, 208-289: per-expert offsets and the tile map ExptData
 * carries), matmul_ogs with gather and the fused SwiGLU, matmul_ogs with gammas, and the scatter-sum of
 * _finalize_matmul (triton_kernels/matmul_ogs_details/_p_matmul_ogs.py:113-495, _finalize_matmul.py:189-378).
 * Weights are bf16 [experts * N, K] row-major: b2_moe_upcast_packed expands the packed MXFP4 layout of the
 * decode-sized path (codes [E][N][Kp/2] with K padded to a multiple of 128, scale blocks
 * [E][ceil(N/128)][Kp/128][512]) into it, exactly.  x [T, hidden] bf16, topk_idx int16 [T,4] (8-byte aligned),
 * topk_w fp32 [T,4] as b2_topk_softmax returns them, b1 fp32 [E][2*intermediate], b2 fp32 [E][hidden] (16-byte
 * aligned), out [T, hidden] bf16.  hidden % 192 == 0 and (2*intermediate) % 192 == 0.  An expert index out of
 * range, or the same expert twice for one token, is dropped and recorded as B2_DEV_BAD_INDEX. */
size_t b2_moe_prefill_workspace_bytes(int64_t tokens, int n_experts, int hidden, int intermediate);
int b2_moe_upcast_packed(const void* codes, const void* scale_blocks, void* out_bf16, int n_experts, int n, int k,
                         void* stream);
int b2_moe_experts_prefill(const void* x, int64_t ldx, const int16_t* topk_idx, const float* topk_w, const void* w1_bf16,
                           const float* b1, const void* w2_bf16, const float* b2, void* out, int64_t ld_out,
                           void* workspace, size_t workspace_bytes, int64_t tokens, int n_experts, int hidden,
                           int intermediate, float alpha, float limit, void* stream);

/* ---- Unembedding for decode: logits and greedy token ---------------------------------
 * logits[b, v] = sum_k hidden[b, k] * weight[v, k] (fp32 accumulation), stored as bf16 when `logits` is
 * given; token_ids[b] (int64, optional) = arg-max over v of the fp32 sums, the smallest v on ties,
 * found per 128-row tile inside the GEMV and reduced over tiles.  Replaces unembedding_decode_forward
 * and unembedding_decode_argmax_forward (tritonllm/gpt_oss/triton/triton_kernels.py:120-198,305-401;
 * callers UnEmbedding.forward / forward_argmax, tritonllm/gpt_oss/triton/model.py:86-116).
 * hidden [batch, hidden_size] bf16 (row stride given), weight [vocab, hidden_size] bf16 contiguous,
 * hidden_size % 64 == 0.  workspace (needed for token_ids): 16-byte aligned,
 * b2_unembed_workspace_bytes(batch, vocab) bytes, need not be zeroed. */
size_t b2_unembed_workspace_bytes(int64_t batch, int vocab);
int b2_unembed_decode(const void* hidden, int64_t hidden_stride_b, const void* weight, void* logits,
                      int64_t logits_stride_b, int64_t* token_ids, void* workspace, size_t workspace_bytes,
                      int64_t batch, int hidden_size, int vocab, void* stream);

/* ---- KV-cache maintenance and the embedding lookup of the decode loop ---------------------
 * The KV store keeps the reference's dense layout: K and V are [batch, n_ctx, kv_heads, head_dim] bf16,
 * contiguous, one position counter for the whole batch (Cache, tritonllm/gpt_oss/triton/model.py:340-433);
 * row_bytes = kv_heads * head_dim * 2, a multiple of 16.
 *
 * b2_kv_slide replaces Cache.slide_window (model.py:391-424): of the `current` tokens held it keeps the
 * newest `keep` (tokens current-keep .. current-1 of every sequence), moves them in place to positions
 * 0 .. keep-1 and zeroes positions keep .. n_ctx-1.  The caller sets its position counter to `keep`.
 * b2_kv_zero_tail replaces the zeroing of Cache.truncate and Cache.reset (model.py:354-371): positions
 * from .. n_ctx-1 of every sequence become zero.
 * b2_embed_gather replaces the torch.nn.Embedding lookup (model.py:896-898, 911): out[t, :] =
 * table[tokens[t], :], tokens int32 or int64 on the device, strides in elements and multiples of 8,
 * hidden % 8 == 0.  A token outside [0, vocab) reads row 0 and records B2_DEV_BAD_INDEX in the device
 * status word. */
int b2_kv_slide(void* k, void* v, int64_t batch, int64_t n_ctx, int64_t row_bytes, int64_t current, int64_t keep,
                void* stream);
int b2_kv_zero_tail(void* k, void* v, int64_t batch, int64_t n_ctx, int64_t row_bytes, int64_t from, void* stream);
int b2_embed_gather(const void* table, int64_t table_stride, const void* tokens, int tokens_are_int64, void* out,
                    int64_t out_stride, int64_t n_tokens, int hidden, int64_t vocab, void* stream);

/* ---- Decode-time front end of the MoE block in one launch ---------------------------------
 * y = RMSNorm(x) (as b2_rmsnorm), logits = bf16(y @ gate) + gate_bias, top-k of the logits by (value
 * descending, expert ascending) with a softmax over the winners, sorted by expert id (as b2_topk_softmax).
 * Replaces self.norm(x) (tritonllm/gpt_oss/triton/model.py:754), the router matmul + bias
 * (tritonllm/gpt_oss/triton/moe.py:46-48, 104-111) and topk(..., apply_softmax=True)
 * (tritonllm/triton_kernels/routing.py:296-297) for decode-sized batches.
 * x, y_out [rows, hidden] bf16 (row strides in elements, multiples of 8; y_out may be x), gain fp32 [hidden],
 * gate_t [n_experts, hidden] bf16 contiguous (the gate weight expert-major), gate_bias fp32 [n_experts] or
 * NULL, logits_out fp32 [rows, n_experts] or NULL, topk_vals fp32 [rows, k], topk_idx int16 [rows, k].
 * hidden % 8 == 0 and <= 3072, n_experts a multiple of 32 up to 128, k <= 4. */
int b2_norm_router_topk(const void* x, int64_t x_stride, const float* gain, const void* gate_t, const float* gate_bias,
                        void* y_out, int64_t y_stride, float* logits_out, int64_t logits_stride, float* topk_vals,
                        int16_t* topk_idx, int64_t rows, int hidden, int n_experts, int k, float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRITONLLM_B200_H */
