/*
 * nemotron_b200.h — C ABI of libnemotron_b200.so
 *
 * B200 (sm_100a) replacements for the bandwidth-bound layer kernels of
 * AIWuXin/nemotron_infer.  Each entry point names the reference host launcher
 * it stands in for (paths are relative to the reference project root; "ops/" is
 * nemotron_infer/csrc/include/ops/).
 *
 * Conventions shared by every entry point
 *   - All pointers are DEVICE pointers owned by the caller; nothing is allocated
 *     or freed here (the reference kernels allocate nothing either; block
 *     workspaces come from the caller's BumpAllocator, tensor/allocator.cuh:58-175).
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default
 *     stream, which is what every reference call site passes (binding.cu:72).
 *   - Calls are asynchronous.  The return value is an nmt_status; NMT_OK means
 *     "validated and enqueued".  The reference returns void and never checks
 *     anything (ops/reduce.cuh:229-244); a non-zero status here means NOTHING
 *     was launched.
 *   - bf16 tensors are row-major, rows contiguous (stride == cols), 16-byte
 *     aligned, and cols % 8 == 0 — the same contract as the reference's
 *     vectorised kernels (ops/reduce.cuh:134-135, ops/elementwise.cuh:198-201).
 *   - rows == 0 / n == 0 is a successful no-op.
 *   - Norm weights are fp32 (model/mlp_block.cuh:76), eps goes inside the rsqrt
 *     after the mean (ops/reduce.cuh:174,438).
 *   - The fp32 vectors of the bf16 entry points (norm weights, conv taps and
 *     bias) are read with 16-byte loads and must be 16-byte aligned; only the
 *     all-fp32 twins (nmt_*_f32) accept 4-byte alignment.  The reference's
 *     BumpAllocator and torch both hand out at least 128-byte alignment
 *     (tensor/allocator.cuh:61,80), so its call sites satisfy this.
 */
#ifndef NEMOTRON_B200_H
#define NEMOTRON_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum nmt_status {
    NMT_OK = 0,
    NMT_ERR_NULL = 1,        /* a required pointer is NULL                        */
    NMT_ERR_ALIGN = 2,       /* a pointer is not aligned as the contract requires */
    NMT_ERR_SHAPE = 3,       /* negative size, cols % 8 != 0, bad group size ...  */
    NMT_ERR_LAUNCH = 4,      /* the CUDA runtime refused the launch               */
    NMT_ERR_UNSUPPORTED = 5, /* shape outside what the kernels cover              */
    NMT_ERR_TOO_LARGE = 6    /* more rows than the built-in scratch of a *_static entry point holds */
} nmt_status;

/* Library identity and status text. */
const char* nmt_version(void);
const char* nmt_status_string(int status);
/* Last CUDA runtime error text recorded by a failed launch on this thread. */
const char* nmt_last_cuda_error(void);

/* Makes `device` current for this library's CUDA runtime instance (the library
 * links the static runtime, so a host that selected its device through another
 * runtime instance should tell this one too). */
int nmt_set_device(int device);
/* cudaDeviceSynchronize(); replaces binding.cu:62 `sync()`. */
int nmt_device_synchronize(void);

/* ---- RMSNorm ------------------------------------------------------------- */

/* y = x * rsqrt(mean(x^2) + eps) * w, fp32.
 * Replaces nemotron::ops::rmsnorm_fp32 (ops/reduce.cuh:113-128).
 * fp32 pointers need 4-byte alignment only; any cols >= 1. */
int nmt_rmsnorm_f32(const float* x, float* y, const float* w,
                    int64_t rows, int64_t cols, float eps, void* stream);

/* Same, bf16 in/out, fp32 accumulation, fp32 weight.
 * Replaces nemotron::ops::rmsnorm_bf16 (ops/reduce.cuh:229-244), which the
 * pybind entry `rmsnorm` calls with cols = 3136 (binding.cu:71-73).
 * y may alias x. */
int nmt_rmsnorm_bf16(const void* x, void* y, const float* w,
                     int64_t rows, int64_t cols, float eps, void* stream);

/* Fused residual add + RMSNorm:
 *     out_res = bf16(x + r)
 *     out     = bf16((out_res * rsqrt(mean(out_res^2) + eps)) * w)
 * Replaces the pair elementwise_ops_bf16<kElementwiseAdd> (ops/elementwise.cuh:
 * 374-419, Add at :241-245) at the tail of one block (model/mlp_block.cuh:104,
 * model/mamba_block.cuh:224, model/attention_block.cuh:210) followed by
 * rmsnorm_bf16 at the head of the next (model/mlp_block.cuh:98,
 * model/mamba_block.cuh:183, model/attention_block.cuh:196, binding.cu:72).
 * The sum of squares is taken over the bf16-ROUNDED sum, exactly what the
 * unfused pair computes.  out_res may alias x or r; out must not alias an input. */
int nmt_add_rmsnorm_bf16(const void* x, const void* r, const float* w,
                         void* out_res, void* out,
                         int64_t rows, int64_t cols, float eps, void* stream);

/* ---- Residual add of block i fused with the pre-norm of block i+1, block code unchanged ------------------ */

/* Every reference block is out = input + mixer(rmsnorm(input)): it opens with rmsnorm_bf16 into its first
 * workspace tensor (model/mlp_block.cuh:98, model/mamba_block.cuh:183, model/attention_block.cuh:196) and closes
 * with the residual add (model/mlp_block.cuh:104, model/mamba_block.cuh:224, model/attention_block.cuh:210), whose
 * output the next block's rmsnorm re-reads at once.  These entry points fuse that pair ACROSS two block calls
 * without changing a block, a binding or a signature.  They have no counterpart in the reference.
 *
 *   nmt_fuse_next_norm(w_next, eps)   called by the orchestrator (engine.py's layer loop) before it calls block i:
 *                                     announces the norm weight of block i+1.  NULL withdraws the announcement.
 *   nmt_block_head_rmsnorm_bf16       what the drop-in rmsnorm_bf16 calls: nmt_rmsnorm_bf16, except that it launches
 *                                     NOTHING when the previous block's fused tail already wrote exactly this tensor
 *                                     (same x, y, w, shape, eps and stream) AND no other entry point of this library
 *                                     has launched a kernel from this thread since that tail.
 *   nmt_block_tail_add_bf16           what the drop-in residual add calls: nmt_add_bf16, except that with a weight
 *                                     announced it launches nmt_add_rmsnorm_bf16 instead and writes rmsnorm(out) *
 *                                     w_next over THIS block's pre-norm tensor (the y of its head call).
 * Requirements, all met by the reference's blocks under engine.py: the block's pre-norm tensor is not read after
 * the block's closing add on that stream (its readers are the block's first projections); the next block's
 * pre-norm tensor has the same address, which the bump allocator guarantees once it is rewound before every layer
 * (engine.py:263, tensor/allocator.cuh:124-129); nothing else writes that address between the two block calls.
 * Whatever does not match runs the plain kernels - same results, one more pass over the rows.  Announce only when
 * the next block really opens with rmsnorm_bf16 on the tensor this block writes (not ahead of a block form that
 * fuses its own norm, nor after the last layer unless the final norm writes into that same workspace).
 * State is per host thread.  nmt_fusion_reset() forgets an announcement and a pending fused tail (call it when a
 * pass is abandoned half way); nmt_fusion_counters reports how many tails were fused and heads skipped. */
int nmt_fuse_next_norm(const float* next_norm_w, float eps);
int nmt_fusion_reset(void);
int nmt_fusion_counters(int64_t* fused_tails, int64_t* elided_heads);
int nmt_block_head_rmsnorm_bf16(const void* x, void* y, const float* w,
                                int64_t rows, int64_t cols, float eps, void* stream);
int nmt_block_tail_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream);

/* ---- Mamba-2 gated RMSNorm ------------------------------------------------ */

/* g = y * silu(z); per group of `group_size` channels:
 *     out = (g * rsqrt(mean_group(g^2) + eps)) * w
 * Replaces nemotron::ops::rmsnorm_gated_bf16<Group> (ops/reduce.cuh:510-527;
 * called at model/mamba_block.cuh:217 with cols = 7680, group_size = 960).
 * The reference's argument order is (in, out, w, gate, ...); here y = in and
 * z = gate.  cols % group_size == 0.  out may alias y or z. */
int nmt_rmsnorm_gated_bf16(const void* y, const void* z, const float* w, void* out,
                           int64_t rows, int64_t cols, int64_t group_size,
                           float eps, void* stream);

/* fp32 twin; replaces nemotron::ops::rmsnorm_gated_fp32<Group>
 * (ops/reduce.cuh:360-377). */
int nmt_rmsnorm_gated_f32(const float* y, const float* z, const float* w, float* out,
                          int64_t rows, int64_t cols, int64_t group_size,
                          float eps, void* stream);

/* ---- Elementwise ----------------------------------------------------------- */

/* out = max(u, 0)^2, bf16 (the fp32 square rounded to nearest even; NaN
 * propagates).  Replaces elementwise_ops_bf16<kElementwiseRelu2>
 * (ops/elementwise.cuh:256-272, launcher :374-419; caller model/mlp_block.cuh:
 * 100).  n = number of elements, n % 8 == 0.  out may alias u. */
int nmt_relu2_bf16(const void* u, void* out, int64_t n, void* stream);

/* fp32 twin of relu2; replaces elementwise_ops_fp32<kElementwiseRelu2>
 * (ops/elementwise.cuh:100-104,177-195).  Any n (scalar tail handled). */
int nmt_relu2_f32(const float* u, float* out, int64_t n, void* stream);

/* out = a + b, bf16 with a single rounding.  Replaces
 * elementwise_ops_bf16<kElementwiseAdd> (ops/elementwise.cuh:241-245).
 * n % 8 == 0.  out may alias a or b. */
int nmt_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream);

/* fp32 twin of add; replaces elementwise_ops_fp32<kElementwiseAdd>
 * (ops/elementwise.cuh:85-89,177-195).  Any n. */
int nmt_add_f32(const float* a, const float* b, float* out, int64_t n, void* stream);

/* ---- Token-embedding gather ------------------------------------------------ */

/* out[i, :] = table[ids[i], :], a bit-exact row copy.
 * Replaces nemotron::ops::embedding_lookup<Hidden> (ops/embedding.cuh:53-66;
 * bound as `embedding` at binding.cu:65-68 with int64 ids, hidden = 3136).
 * hidden % 8 == 0.  The reference never range-checks an id; here an id outside
 * [0, vocab) is never dereferenced: its output row is zero-filled and, when
 * err_flag != NULL, *err_flag (device int32) is set to 1.  Pass vocab <= 0 to
 * disable the check (the reference's behaviour). */
int nmt_embedding_bf16_i64(const void* table, const int64_t* ids, void* out,
                           int64_t num_tokens, int64_t hidden, int64_t vocab,
                           int32_t* err_flag, void* stream);
int nmt_embedding_bf16_i32(const void* table, const int32_t* ids, void* out,
                           int64_t num_tokens, int64_t hidden, int64_t vocab,
                           int32_t* err_flag, void* stream);

/* ---- Mamba-2 causal conv1d + SiLU (with the x | B | C split) -------------------- */

/* y[b, t, c] = silu(bias[c] + sum_k w[c, k] * xbc[b, t - 3 + k, c]), k = 0..3, zero before t = 0; bf16 in/out,
 * fp32 taps, bias and accumulation.  Replaces nemotron::ops::mamba2::causal_conv1d_prefill_bf16
 * (ops/mamba2/causal_conv1d.cuh:369-389) TOGETHER WITH the three strided copies that split its output
 * (model/mamba_block.cuh:199-207): channels [0, n0) are written to out0 as a contiguous [batch*S, n0] tensor,
 * [n0, n0+n1) to out1, the rest to out2.  Pass n1 = n2 = 0 (out1 = out2 = NULL) for the unsplit
 * [batch*S, conv_dim] output of the reference.  n0, n1, n2 multiples of 8.  state_out (may be NULL) receives the
 * last three raw inputs per channel, [batch, conv_dim, 3] fp32, the layout the decode step continues from. */
int nmt_causal_conv1d_silu_split_bf16(const void* xbc, const float* w, const float* bias, void* out0, void* out1,
                                      void* out2, int64_t n0, int64_t n1, int64_t n2, float* state_out,
                                      int64_t S, int64_t batch, void* stream);

/* The single-token step of the same op: xbc is [batch, conv_dim] bf16 (one new row per sequence), state is the
 * [batch, conv_dim, 3] fp32 window (read, shifted, written back - the tensor the prefill call leaves in
 * state_out), the output goes straight into the x | B | C tensors ([batch, n_i] each).  Replaces
 * causal_conv1d_decode_bf16 (ops/mamba2/causal_conv1d.cuh:391-456) and the three strided copies after it
 * (model/mamba_block.cuh:487-497).  state must be 16-byte aligned. */
int nmt_causal_conv1d_silu_decode_split_bf16(const void* xbc, const float* w, const float* bias, void* out0, void* out1,
                                             void* out2, int64_t n0, int64_t n1, int64_t n2, float* state, int64_t batch,
                                             void* stream);

/* The Mamba-2 state-space recurrence for ONE token per sequence, the step between the conv step and the gated norm
 * of the decode block (model/mamba_block.cuh:298-301, 499-502).  Replaces the kernel ssm_decode_bf16<H, D, N>
 * (ops/mamba2/ssm.cuh:43-103, launched there as <<<batch * H, 128>>>), same arguments in the same order:
 *   dt' = clamp(softplus(dt[h] + dt_bias[h]), dt_min, dt_max),  dA = exp(-exp(A_log[h]) * dt')
 *   state[b, h, p, n] = state * dA + dt' * B[b, g, n] * x[b, h, p]     (fp32, updated in place)
 *   y[b, h, p] = sum_n state[b, h, p, n] * C[b, g, n] + D[h] * x[b, h, p],   g = h / (heads / n_groups)
 * x, y [batch, heads * head_dim] bf16; dt [batch, heads] bf16; B, C [batch, n_groups, state_size] bf16; A_log, D,
 * dt_bias (may be NULL) [heads] fp32; state [batch, heads, head_dim, state_size] fp32.  state_size <= 256.
 * State and y are bit-identical to the reference kernel's (same element-to-lane assignment, same reduction tree).
 * The state rows are requested before the kernel waits for its predecessor on the stream: that predecessor must
 * not be the one that writes `state` (in the decode block it is the conv step; the state's only writer is this
 * entry point one token earlier). */
int nmt_ssm_decode_step_bf16(const void* x, const void* dt, const float* A_log, const void* B, const void* C,
                             const float* D, const float* dt_bias, float* state, void* y, int64_t batch, int64_t heads,
                             int64_t head_dim, int64_t state_size, int64_t n_groups, float dt_min, float dt_max,
                             void* stream);

/* Attention for ONE query token per call over the KV cache, the decode step of the attention block
 * (model/attention_block.cuh:249-253, 403-406).  Replaces sdpa_decode_bf16<128> (ops/attention/sdpa_decode.cuh:
 * 275-291: its split kernel :56-122, combine kernel :127-186 and the process-wide scratch :192-221), same arguments
 * plus the workspace:
 *   O[h] = sum_{s < S_cache} softmax_s(Q[h] . K_cache[g, s] / sqrt(128)) V_cache[g, s],   g = h / (heads / kv_heads),
 *   then K_new / V_new [kv_heads, 128] are written to position S_cache of the caches [kv_heads, total_S, 128] - the
 *   new token does not attend to itself, exactly as in the reference.  S_cache == 0 gives O = 0.
 * All tensors bf16; Q and O [heads, 128]; fp32 accumulation; results agree with the reference kernel to bf16
 * rounding (the positions are split differently, so the fp32 sums associate differently).  head_dim must be 128 and
 * heads / kv_heads one of 1, 2, 4, 5, 8 (NMT_ERR_UNSUPPORTED otherwise).  workspace: nmt_sdpa_decode_workspace_bytes(
 * S_cache, heads) bytes of device memory, 16-byte aligned, contents need no initialisation.  Q, the caches 8-byte
 * aligned.  Two launches. */
int64_t nmt_sdpa_decode_workspace_bytes(int64_t S_cache, int64_t num_heads);
int nmt_sdpa_decode_bf16(const void* Q, void* K_cache, void* V_cache, void* O, const void* K_new, const void* V_new,
                         int64_t S_cache, int64_t total_S, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                         void* workspace, void* stream);

/* fp32 twin, unsplit; replaces causal_conv1d_prefill_fp32 (ops/mamba2/causal_conv1d.cuh:115-127). */
int nmt_causal_conv1d_silu_f32(const float* x, const float* w, const float* bias, float* y, float* state_out,
                               int64_t conv_dim, int64_t S, int64_t batch, void* stream);

/* ---- W8A16 GEMV (single-token decode projections) --------------------------------- */

/* y[n] = bf16((sum_k e4m3(W[n,k]) * bf16(x[k])) * w_scale[n]), fp32 accumulation.  Replaces
 * nemotron::ops::gemv_fp8 (ops/gemv.cuh:87-104; kernel :48-85), same arguments: W is [N, K] row-major e4m3 with
 * one fp32 scale per output row, x is K bf16 activations.  K % 16 == 0, W 16-byte aligned.
 * When K % 64 == 0 the products run on tensor cores with x held as f16 times a power of two taken from max|x|:
 * exact for elements within 2^-28 of the maximum (nmt_tune_set("gemv.variant", 1) keeps fp32 products).
 * Ordering contract: W and w_scale are model constants to this kernel -- its first weight loads are issued
 * before it waits for the kernel that precedes it on the stream (programmatic dependent launch), so that
 * preceding kernel must not be the one that writes W or w_scale (an on-the-fly weight quantiser, a staging
 * copy kernel).  Put any other kernel, an event or a stream synchronisation between such a producer and this
 * call, or switch the overlap off with nmt_tune_set("launch.pdl", 2).  x, the norm weight and the residual have
 * no such restriction: they are read after the wait. */
int nmt_gemv_w8a16(const void* x_bf16, const void* W_e4m3, const float* w_scale, void* y_bf16, int64_t N, int64_t K,
                   void* stream);

/* The same product with the decode block's neighbours folded in, one launch instead of up to four:
 *   norm_w != NULL      x is first replaced by rmsnorm(x) * norm_w (eps as given), the pre-norm of
 *                       mlp_block_forward_fp8 (model/mlp_block.cuh:140) and mamba_block_decode_fp8
 *                       (model/mamba_block.cuh:473); x must then be 16-byte aligned;
 *   activation == 1     y = relu(y)^2 on the bf16 result, the step between up_proj and down_proj
 *                       (model/mlp_block.cuh:145-147);
 *   residual != NULL    y[n] += residual[n] in bf16, the block's closing add (model/mlp_block.cuh:170-172,
 *                       model/mamba_block.cuh:512-514).
 * Byte-identical to nmt_rmsnorm_bf16 -> nmt_gemv_w8a16 -> nmt_relu2_bf16 / nmt_add_bf16 with this library's
 * defaults.  K % 64 == 0, and K <= 10240 when norm_w is given (NMT_ERR_UNSUPPORTED otherwise: there is no unfused fallback inside,
 * it would need scratch memory).  y may alias residual (each element is read, then written, by one thread) but
 * not x.  Mamba's three in_proj slices (model/mamba_block.cuh:476-481) are one call
 * with N = INTER + CONV_DIM + H rows, since they are consecutive rows of one matrix. */
int nmt_gemv_w8a16_fused(const void* x_bf16, const float* norm_w, float eps, const void* W_e4m3, const float* w_scale,
                         int activation, const void* residual_bf16, void* y_bf16, int64_t N, int64_t K, void* stream);

/* The in_proj of the Mamba-2 decode block with the pre-norm in front of it and the single-token conv step behind it
 * (model/mamba_block.cuh:473-497: rmsnorm_bf16, three gemv_fp8 over consecutive rows of one matrix,
 * causal_conv1d_decode_bf16, three strided copies) in one launch.  As nmt_gemv_w8a16_fused(x, norm_w, eps, W, w_scale,
 * 0, NULL, y, N, K), except that the output rows [conv_row_lo, conv_row_lo + n0 + n1 + n2) - the xBC channels - are not
 * stored in y: each goes, rounded to bf16 as it would have been stored, through the conv step of its channel (conv_w
 * [channels][4], conv_bias [channels], window conv_state [channels][3] fp32 updated in place: one sequence) and SiLU,
 * and lands in out0 [n0] | out1 [n1] | out2 [n2].  Byte-identical to nmt_gemv_w8a16_fused followed by
 * nmt_causal_conv1d_silu_decode_split_bf16 with batch 1.  The other rows (gate, dt) are stored in y as usual.
 * K % 64 == 0, K <= 10240 with norm_w; conv_w 16-byte aligned. */
int nmt_gemv_w8a16_fused_conv_step(const void* x_bf16, const float* norm_w, float eps, const void* W_e4m3, const float* w_scale,
                                   void* y_bf16, int64_t N, int64_t K, int64_t conv_row_lo, const float* conv_w,
                                   const float* conv_bias, float* conv_state, void* out0, void* out1, void* out2, int64_t n0,
                                   int64_t n1, int64_t n2, void* stream);

/* The out_proj of the Mamba-2 decode block with the gated RMSNorm in front of it and the residual add behind it
 * (model/mamba_block.cuh:504-514: rmsnorm_gated_bf16, gemv_fp8, elementwise add) in one launch:
 *     out = W @ (gated_rmsnorm(y_in, gate, group_size) * gnorm_w) * w_scale  (+ residual)
 * Byte-identical to nmt_rmsnorm_gated_bf16 -> nmt_gemv_w8a16_fused(residual) with this library's defaults: every CTA
 * normalises its own copy of the row, one warp per group, in the stand-alone kernel's order.  y_in, gate bf16 [K],
 * 16-byte aligned; gnorm_w fp32 [K], 16-byte aligned; K % 64 == 0, K <= 10240, group_size % 8 == 0 and <= 2048,
 * K % group_size == 0 (NMT_ERR_UNSUPPORTED / NMT_ERR_SHAPE otherwise).  residual may be NULL; out may alias it. */
int nmt_gemv_w8a16_gated(const void* y_in_bf16, const void* gate_bf16, const float* gnorm_w, float eps, int64_t group_size,
                         const void* W_e4m3, const float* w_scale, const void* residual_bf16, void* out_bf16, int64_t N,
                         int64_t K, void* stream);

/* ---- Per-tensor FP8 (e4m3) activation quantisation ---------------------------- */

/* out_fp8 = e4m3(clamp(x / s, +-448)), s = max|x| / 448 (1/448 for an all-zero tensor), *scale_out = s.
 * Replaces nemotron::ops::quantize_activation_fp8 (ops/gemm.cuh:291-307: fp8_amax_kernel :257-273 and
 * fp8_quant_kernel :275-289), same arguments: `amax_scratch` is one device uint32 the call clears and uses.
 * n % 8 == 0; x 16-byte, out 8-byte aligned.  scale_out may be NULL. */
int nmt_quantize_fp8(const void* x_bf16, void* out_fp8, float* scale_out, unsigned int* amax_scratch,
                     int64_t n, void* stream);

/* relu^2 fused with the quantisation that follows it in the FP8 MLP block (model/mlp_block.cuh:163-168):
 * out_fp8 = quantize(bf16(max(u,0)^2)) without ever writing the bf16 activation tensor. */
int nmt_relu2_quant_fp8(const void* u_bf16, void* out_fp8, float* scale_out, unsigned int* amax_scratch,
                        int64_t n, void* stream);

/* Device workspace the two entry points below need for `rows` rows (one uint32 for the running maximum
 * plus one float per row for its rstd); 16-byte aligned, caller-owned, contents need no initialisation. */
int64_t nmt_fp8_workspace_bytes(int64_t rows);

/* RMSNorm fused with the quantisation of its output (model/mlp_block.cuh:140,158; mamba_block.cuh:378-381;
 * attention_block.cuh:328-330): out_fp8 = quantize(rmsnorm_bf16(x, w)), the bf16 normed tensor is never
 * materialised.  cols % 8 == 0, cols <= 32768. */
int nmt_rmsnorm_quant_fp8(const void* x, const float* w, void* out_fp8, float* scale_out, void* workspace,
                          int64_t rows, int64_t cols, float eps, void* stream);

/* The same with the preceding residual add: out_res = bf16(x + r), out_fp8 = quantize(rmsnorm_bf16(out_res, w)).
 * out_res may alias x or r. */
int nmt_add_rmsnorm_quant_fp8(const void* x, const void* r, const float* w, void* out_res, void* out_fp8,
                              float* scale_out, void* workspace, int64_t rows, int64_t cols, float eps,
                              void* stream);

/* Gated RMSNorm fused with the maximum its quantiser needs (the FP8 Mamba block quantises the gated norm's
 * output right away, model/mamba_block.cuh:415-419): out_bf16 = rmsnorm_gated_bf16(y, z, w) as usual, and
 * out_fp8 / *scale_out = quantize(out_bf16) without a separate maximum pass over out_bf16.
 * `amax_scratch` is one device uint32, as in nmt_quantize_fp8. */
int nmt_rmsnorm_gated_quant_fp8(const void* y, const void* z, const float* w, void* out_bf16, void* out_fp8,
                                float* scale_out, unsigned int* amax_scratch, int64_t rows, int64_t cols,
                                int64_t group_size, float eps, void* stream);

/* nmt_add_rmsnorm_quant_fp8 for callers that cannot provide the workspace.  This entry point has no
 * counterpart in the reference.
 *
 * Who needs it: a host that must not, or cannot, allocate device memory at the point of the call -- the
 * reference's engine bans cudaMalloc/cudaFree inside its per-layer loop because cudaFree stalls the device
 * (ops/gemm.cuh:322-323, binding.cu:58); a minimal foreign-function binding only relays the tensor addresses it is given and
 * has no device allocator; a server that has already committed all free memory to its caches cannot rely on a
 * late allocation succeeding.  Here the workspace is a fixed array inside the library image instead.
 *
 * Same arguments and results as nmt_add_rmsnorm_quant_fp8 minus `workspace`; the call performs no allocation
 * of any kind (host or device).  Limits and rules:
 *   - rows <= NMT_STATIC_SCRATCH_MAX_ROWS, else NMT_ERR_TOO_LARGE is returned and nothing is launched.  The
 *     array is 256 + 4 * NMT_STATIC_SCRATCH_MAX_ROWS bytes and is resident on every GPU that loads the library
 *     for the life of the process.
 *   - The first call on each device looks up the array's device address (with that device current) and caches
 *     it; make that first call outside any stream capture.  The cached address stays valid until that device
 *     is reset (cudaDeviceReset); a process that resets a device must not call this entry point on it again.
 *   - All calls on a device share the one array.  Calls are safe back to back on one stream (each call resets
 *     what it needs); two calls whose kernels can overlap on the GPU (different streams, no ordering between
 *     them) race on the array and give wrong results -- order them, or use the workspace form for one. */
#define NMT_STATIC_SCRATCH_MAX_ROWS 65536
int nmt_add_rmsnorm_quant_fp8_static(const void* x, const void* r, const float* w, void* out_res, void* out_fp8,
                                     float* scale_out, int64_t rows, int64_t cols, float eps, void* stream);

/* ---- Test and tuning hooks -------------------------------------------------- */

/* Selects a kernel variant / launch shape by name (for measurement sweeps).
 * Unknown keys return NMT_ERR_UNSUPPORTED.  Not needed in normal use: the
 * defaults are the measured-best settings. */
int nmt_tune_set(const char* key, int value);
int nmt_tune_get(const char* key, int* value);
/* The staged (TMA) kernels bound every mbarrier wait; a wait that runs out is counted on the device and the
 * kernel winds down instead of spinning.  Returns the number of such timeouts on the current device since
 * load (synchronises the device; 0 in a healthy run, -1 if the counter cannot be read). */
int64_t nmt_device_wait_timeouts(void);
/* Exercises that path without involving a product kernel: one thread of a 32-thread CTA waits, for at most `polls`
 * polls (1..4096), on an mbarrier in its own shared memory that nothing will ever complete.  The wait gives up after
 * microseconds, nmt_device_wait_timeouts() rises by one, *gave_up_device (device int32, may be NULL) is set to 1, and
 * the context stays usable.  Has no counterpart in the reference. */
int nmt_selftest_wait_runs_out(int polls, int* gave_up_device, void* stream);
/* Number of kernel launches this library has enqueued since load (all threads). */
int64_t nmt_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NEMOTRON_B200_H */
