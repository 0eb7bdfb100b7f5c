// The reference's blocks with the steps around their GEMMs collapsed onto this library's fused entry points.
//
// How to use.  Give the compiler this directory's parent first on the include path and make this header the first
// thing a translation unit sees (nvcc --pre-include .../nemotron_b200_shim/model/blocks_b200.cuh, or an #include
// ahead of the reference's headers).  It pulls in the reference's model/*.cuh itself, so binding.cu, the block
// tests and engine.py stay as they are, and afterwards
//   - every RMSNorm, gated RMSNorm, relu^2, residual add, embedding gather and W8A16 GEMV call of the reference
//     lands on libnemotron_b200.so (ops/{reduce,elementwise,embedding,gemv}.cuh of this directory);
//   - nemotron::ops::quantize_activation_fp8 (ops/gemm.cuh:291-307) forwards to nmt_quantize_fp8; the reference's
//     own stays reachable as quantize_activation_fp8_reference;
//   - the block entry points listed below are the fused forms defined in this file, under the reference's own
//     names and signatures; the reference's originals stay reachable with the suffix _reference (used by the
//     tests for side-by-side runs, and by the fused forms themselves for the cases they do not cover).
//
//   mlp_block_forward_fp8      (model/mlp_block.cuh:122-178)  prefill: norm -> quantise and relu^2 -> quantise are one
//                              entry point each (:140+158, :163+167); single token: norm + up_proj + relu^2 is one
//                              launch, down_proj + residual add another (:140-148, :170-173) - 2 launches for 5
//   mamba_block_forward_bf16   (model/mamba_block.cuh:149-227) conv1d + SiLU writes x | B | C directly (:195-207)
//   mamba_block_decode_bf16    (model/mamba_block.cuh:238-311) the same for the single-token conv step (:281-293); the
//                              state-space step on nmt_ssm_decode_step_bf16 (:298-301)
//   mamba_block_forward_fp8    (model/mamba_block.cuh:336-429) norm -> quantise (:378-381), conv + split (:394-406),
//                              gated norm -> quantise (:415-420)
//   mamba_block_decode_fp8     (model/mamba_block.cuh:439-516) norm + the three in_proj slices in one launch
//                              (:473-481), conv step + split (:484-496), the state-space step on
//                              nmt_ssm_decode_step_bf16 (:499-502), out_proj + residual add (:508-514) -
//                              5 launches for 12
//   attention_block_forward_fp8 (model/attention_block.cuh:286-358) norm -> quantise in one entry point (:328-330)
//   attention_block_decode_fp8  (model/attention_block.cuh:363-414) the pre-norm inside each of the q / k / v GEMVs
//                              (:396-401), o_proj + residual add in one launch (:408-413) - 4 launches of this
//                              library for 6
//   - nemotron::ops::attention::sdpa_decode_bf16 (ops/attention/sdpa_decode.cuh:275-291), called by both decode forms
//     of the attention block (model/attention_block.cuh:251, 405), forwards to nmt_sdpa_decode_bf16;
// Every fused form returns what the reference's sequence of this library's single ops returns, byte for byte
// (the entry points are tested for exactly that), so swapping a block changes its traffic, not its numbers.
#ifndef NEMOTRON_B200_SHIM_BLOCKS_CUH
#define NEMOTRON_B200_SHIM_BLOCKS_CUH

#include <cfloat>
#include <cstddef>
#include <cstdint>

#include "../ops/reduce.cuh"
#include "../ops/elementwise.cuh"
#include "../ops/embedding.cuh"
#include "../ops/gemv.cuh"

// -- the reference's quantiser under another name, ours under its name ------------------------------------------
#define quantize_activation_fp8 quantize_activation_fp8_reference
#include "ops/gemm.cuh"
#undef quantize_activation_fp8

namespace nemotron::ops {
inline void quantize_activation_fp8(const __nv_bfloat16* x_bf16, __nv_fp8_e4m3* x_fp8, float* x_scale,
                                    unsigned int* amax_scratch, size_t n, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_quantize_fp8(x_bf16, x_fp8, x_scale, amax_scratch, static_cast<int64_t>(n), stream),
                           "nmt_quantize_fp8");
}
}  // namespace nemotron::ops

// -- the reference's decode attention under another name, ours under its name (defined after the allocator) -----
#define sdpa_decode_bf16 sdpa_decode_bf16_reference
#include "ops/attention/sdpa_decode.cuh"
#undef sdpa_decode_bf16

// -- the reference's blocks; the seven that get a fused form keep their bodies under *_reference ------------------
#define mlp_block_forward_fp8 mlp_block_forward_fp8_reference
#define mamba_block_forward_bf16 mamba_block_forward_bf16_reference
#define mamba_block_decode_bf16 mamba_block_decode_bf16_reference
#define mamba_block_forward_fp8 mamba_block_forward_fp8_reference
#define mamba_block_decode_fp8 mamba_block_decode_fp8_reference
#define attention_block_forward_fp8 attention_block_forward_fp8_reference
#define attention_block_decode_fp8 attention_block_decode_fp8_reference
#include "tensor/tensor.h"
#include "tensor/allocator.cuh"

namespace nemotron::ops::attention {
// ops/attention/sdpa_decode.cuh:275-291, same arguments.  The partial results of the splits live in a transient tensor
// of the caller's bump allocator (the reference keeps a process-wide cudaMalloc'd scratch for them, :192-221).
template <int HEAD = 128>
inline void sdpa_decode_bf16(const __nv_bfloat16* Q, __nv_bfloat16* K_cache, __nv_bfloat16* V_cache, __nv_bfloat16* O,
                             const __nv_bfloat16* K_new, const __nv_bfloat16* V_new, const int S_cache, const int total_S,
                             const int num_heads, int num_kv_heads = -1, cudaStream_t stream = nullptr) {
    if (num_heads == 0) return;
    if (num_kv_heads <= 0) num_kv_heads = num_heads;
    const int64_t bytes = nmt_sdpa_decode_workspace_bytes(S_cache, num_heads);
    void* ws = bytes > 0 ? nemotron::allocate_tensor<float>(nemotron::TensorShape::make_1d(bytes / 4)).data_ : nullptr;
    const int s = nmt_sdpa_decode_bf16(Q, K_cache, V_cache, O, K_new, V_new, S_cache, total_S, num_heads, num_kv_heads, HEAD, ws, stream);
    if (s == NMT_ERR_UNSUPPORTED)                                  // a head size or group ratio this library has no kernel for
        return sdpa_decode_bf16_reference<HEAD>(Q, K_cache, V_cache, O, K_new, V_new, S_cache, total_S, num_heads, num_kv_heads, stream);
    nemotron::ops::detail::nmt_shim_check(s, "nmt_sdpa_decode_bf16");
}
}  // namespace nemotron::ops::attention

#include "model/mlp_block.cuh"
#include "model/mamba_block.cuh"
#include "model/attention_block.cuh"
#undef mlp_block_forward_fp8
#undef mamba_block_forward_bf16
#undef mamba_block_decode_bf16
#undef mamba_block_forward_fp8
#undef mamba_block_decode_fp8
#undef attention_block_forward_fp8
#undef attention_block_decode_fp8

namespace nemotron::model {

namespace b200 {
using bf16 = __nv_bfloat16;
using fp8 = __nv_fp8_e4m3;
inline void ok(int status, const char* what) { nemotron::ops::detail::nmt_shim_check(status, what); }
// Transient tensors come from the caller's bump allocator, as in the reference's blocks (tensor/allocator.cuh:203-213).
template <typename T>
inline T* scratch(int64_t n) { return allocate_tensor<T>(TensorShape::make_1d(n)).data_; }
constexpr size_t kLtWorkspace = 32ull * 1024 * 1024;      // cuBLASLt workspace, the reference's size (model/mlp_block.cuh:132)
// x | B | C widths of the Mamba-2 conv output must be whole 16-byte vectors for the split-fused conv.
constexpr bool split_ok(int inter, int gn) { return inter % 8 == 0 && gn % 8 == 0; }
}  // namespace b200

// ---------------------------------------------------------------------------------------------------------------
// MLP, FP8 weights
// ---------------------------------------------------------------------------------------------------------------
template <int HIDDEN, int INTER>
inline void mlp_block_forward_fp8(const __nv_bfloat16* input, const MLPBlockWeightsFP8& w, __nv_bfloat16* out, int M,
                                  cudaStream_t stream = nullptr) {
    using namespace b200;
    constexpr float EPS = 1e-5f;
    if (M <= 0) return;
    if (M == 1) {
        if constexpr (HIDDEN % 64 == 0 && INTER % 64 == 0 && HIDDEN <= 10240) {
            bf16* act = scratch<bf16>(INTER);
            ok(nmt_gemv_w8a16_fused(input, w.block_norm_w, EPS, w.up_proj_w, w.up_proj_wscale, /*relu^2*/ 1, nullptr, act,
                                    INTER, HIDDEN, stream), "nmt_gemv_w8a16_fused(norm, up_proj, relu2)");
            ok(nmt_gemv_w8a16_fused(act, nullptr, 0.f, w.down_proj_w, w.down_proj_wscale, 0, input, out, HIDDEN, INTER,
                                    stream), "nmt_gemv_w8a16_fused(down_proj, residual)");
            return;
        } else {
            return mlp_block_forward_fp8_reference<HIDDEN, INTER>(input, w, out, M, stream);
        }
    }
    const size_t rows = static_cast<size_t>(M);
    fp8* norm_q = scratch<fp8>(rows * HIDDEN);
    bf16* up = scratch<bf16>(rows * INTER);
    fp8* act_q = scratch<fp8>(rows * INTER);
    bf16* down = scratch<bf16>(rows * HIDDEN);
    float* scales = scratch<float>(2);
    unsigned int* amax = scratch<unsigned int>(1);
    char* stats = scratch<char>(nmt_fp8_workspace_bytes(M));
    char* lt = scratch<char>(static_cast<int64_t>(kLtWorkspace));
    ok(nmt_rmsnorm_quant_fp8(input, w.block_norm_w, norm_q, scales, stats, M, HIDDEN, EPS, stream), "nmt_rmsnorm_quant_fp8");
    ops::gemm_fp8(norm_q, w.up_proj_w, up, scales, w.up_proj_wscale, M, INTER, HIDDEN, lt, kLtWorkspace, stream);
    ok(nmt_relu2_quant_fp8(up, act_q, scales + 1, amax, static_cast<int64_t>(rows * INTER), stream), "nmt_relu2_quant_fp8");
    ops::gemm_fp8(act_q, w.down_proj_w, down, scales + 1, w.down_proj_wscale, M, HIDDEN, INTER, lt, kLtWorkspace, stream);
    ops::elementwise_ops_bf16<ops::kElementwiseAdd>(input, down, out, rows * HIDDEN, 1.f, nullptr, 0.f, 1.f, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Mamba-2.  Shared middle of the two prefill forms: conv1d + SiLU straight into x | B | C, scan, (gated norm by caller)
// ---------------------------------------------------------------------------------------------------------------
template <int HIDDEN, int H, int P, int N, int G, int CONV_K = 4>
inline void mamba_block_forward_bf16(const __nv_bfloat16* input, const Mamba2BlockWeightsBF16& w, __nv_bfloat16* out,
                                     int B, int S, float* conv_state_out = nullptr, float* ssm_state_out = nullptr,
                                     cudaStream_t stream = nullptr) {
    using namespace b200;
    constexpr int INTER = H * P, GN = G * N, CONV_DIM = INTER + 2 * GN;
    constexpr float EPS = 1e-5f;
    if constexpr (!split_ok(INTER, GN) || CONV_K != 4) {
        return mamba_block_forward_bf16_reference<HIDDEN, H, P, N, G, CONV_K>(input, w, out, B, S, conv_state_out, ssm_state_out, stream);
    } else {
        const int M = B * S;
        if (M <= 0) return;
        const size_t rows = static_cast<size_t>(M);
        bf16* normed = scratch<bf16>(rows * HIDDEN);         // first allocation, like the reference: the cross-block fusion relies on it
        bf16* gate = scratch<bf16>(rows * INTER);
        bf16* xbc = scratch<bf16>(rows * CONV_DIM);
        bf16* dt = scratch<bf16>(rows * H);
        bf16* x = scratch<bf16>(rows * INTER);
        bf16* Bm = scratch<bf16>(rows * GN);
        bf16* Cm = scratch<bf16>(rows * GN);
        bf16* y = scratch<bf16>(rows * INTER);
        bf16* gnormed = scratch<bf16>(rows * INTER);
        bf16* mixer = scratch<bf16>(rows * HIDDEN);
        ops::rmsnorm_bf16(input, normed, w.block_norm_w, M, HIDDEN, EPS, stream);
        ops::gemm_bf16(normed, w.in_proj_w, gate, M, INTER, HIDDEN, stream);
        ops::gemm_bf16(normed, w.in_proj_w + static_cast<size_t>(INTER) * HIDDEN, xbc, M, CONV_DIM, HIDDEN, stream);
        ops::gemm_bf16(normed, w.in_proj_w + static_cast<size_t>(INTER + CONV_DIM) * HIDDEN, dt, M, H, HIDDEN, stream);
        ok(nmt_causal_conv1d_silu_split_bf16(xbc, w.conv1d_w, w.conv1d_b, x, Bm, Cm, INTER, GN, GN, conv_state_out, S, B, stream),
           "nmt_causal_conv1d_silu_split_bf16");
        ops::mamba2::ssd_scan_chunked_prefill_bf16<H, P, N, 128>(x, dt, w.A_log, Bm, Cm, w.D, w.dt_bias, y, ssm_state_out, B, S, G,
                                                                 0.f, FLT_MAX, stream);
        ops::rmsnorm_gated_bf16<G>(y, gnormed, w.gnorm_w, gate, M, INTER, INTER / G, EPS, stream);
        ops::gemm_bf16(gnormed, w.out_proj_w, mixer, M, HIDDEN, INTER, stream);
        ops::elementwise_ops_bf16<ops::kElementwiseAdd>(input, mixer, out, rows * HIDDEN, 1.f, nullptr, 0.f, 1.f, stream);
    }
}

template <int HIDDEN, int H, int P, int N, int G, int CONV_K = 4>
inline void mamba_block_decode_bf16(const __nv_bfloat16* input, const Mamba2BlockWeightsBF16& w, float* conv_state,
                                    float* ssm_state, __nv_bfloat16* out, int B, cudaStream_t stream = nullptr) {
    using namespace b200;
    constexpr int INTER = H * P, GN = G * N, CONV_DIM = INTER + 2 * GN;
    constexpr float EPS = 1e-5f;
    if constexpr (!split_ok(INTER, GN) || CONV_K != 4) {
        return mamba_block_decode_bf16_reference<HIDDEN, H, P, N, G, CONV_K>(input, w, conv_state, ssm_state, out, B, stream);
    } else {
        if (B <= 0) return;
        const size_t rows = static_cast<size_t>(B);
        bf16* normed = scratch<bf16>(rows * HIDDEN);
        bf16* gate = scratch<bf16>(rows * INTER);
        bf16* xbc = scratch<bf16>(rows * CONV_DIM);
        bf16* dt = scratch<bf16>(rows * H);
        bf16* x = scratch<bf16>(rows * INTER);
        bf16* Bm = scratch<bf16>(rows * GN);
        bf16* Cm = scratch<bf16>(rows * GN);
        bf16* y = scratch<bf16>(rows * INTER);
        bf16* gnormed = scratch<bf16>(rows * INTER);
        bf16* mixer = scratch<bf16>(rows * HIDDEN);
        ops::rmsnorm_bf16(input, normed, w.block_norm_w, B, HIDDEN, EPS, stream);
        ops::gemm_bf16(normed, w.in_proj_w, gate, B, INTER, HIDDEN, stream);
        ops::gemm_bf16(normed, w.in_proj_w + static_cast<size_t>(INTER) * HIDDEN, xbc, B, CONV_DIM, HIDDEN, stream);
        ops::gemm_bf16(normed, w.in_proj_w + static_cast<size_t>(INTER + CONV_DIM) * HIDDEN, dt, B, H, HIDDEN, stream);
        ok(nmt_causal_conv1d_silu_decode_split_bf16(xbc, w.conv1d_w, w.conv1d_b, x, Bm, Cm, INTER, GN, GN, conv_state, B, stream),
           "nmt_causal_conv1d_silu_decode_split_bf16");
        ok(nmt_ssm_decode_step_bf16(x, dt, w.A_log, Bm, Cm, w.D, w.dt_bias, ssm_state, y, B, H, P, N, G, 0.f, FLT_MAX, stream),
           "nmt_ssm_decode_step_bf16");
        ops::rmsnorm_gated_bf16<G>(y, gnormed, w.gnorm_w, gate, B, INTER, INTER / G, EPS, stream);
        ops::gemm_bf16(gnormed, w.out_proj_w, mixer, B, HIDDEN, INTER, stream);
        ops::elementwise_ops_bf16<ops::kElementwiseAdd>(input, mixer, out, rows * HIDDEN, 1.f, nullptr, 0.f, 1.f, stream);
    }
}

template <int HIDDEN, int H, int P, int N, int G, int CONV_K = 4>
inline void mamba_block_forward_fp8(const __nv_bfloat16* input, const Mamba2BlockWeightsFP8& w, __nv_bfloat16* out, int B,
                                    int S, float* conv_state_out = nullptr, float* ssm_state_out = nullptr,
                                    cudaStream_t stream = nullptr) {
    using namespace b200;
    constexpr int INTER = H * P, GN = G * N, CONV_DIM = INTER + 2 * GN;
    constexpr float EPS = 1e-5f;
    if constexpr (!split_ok(INTER, GN) || CONV_K != 4) {
        return mamba_block_forward_fp8_reference<HIDDEN, H, P, N, G, CONV_K>(input, w, out, B, S, conv_state_out, ssm_state_out, stream);
    } else {
        const int M = B * S;
        if (M <= 0) return;
        const size_t rows = static_cast<size_t>(M);
        fp8* norm_q = scratch<fp8>(rows * HIDDEN);
        bf16* gate = scratch<bf16>(rows * INTER);
        bf16* xbc = scratch<bf16>(rows * CONV_DIM);
        bf16* dt = scratch<bf16>(rows * H);
        bf16* x = scratch<bf16>(rows * INTER);
        bf16* Bm = scratch<bf16>(rows * GN);
        bf16* Cm = scratch<bf16>(rows * GN);
        bf16* y = scratch<bf16>(rows * INTER);
        bf16* gnormed = scratch<bf16>(rows * INTER);
        fp8* gnorm_q = scratch<fp8>(rows * INTER);
        bf16* mixer = scratch<bf16>(rows * HIDDEN);
        float* scales = scratch<float>(2);
        unsigned int* amax = scratch<unsigned int>(1);
        char* stats = scratch<char>(nmt_fp8_workspace_bytes(M));
        char* lt = scratch<char>(static_cast<int64_t>(kLtWorkspace));
        ok(nmt_rmsnorm_quant_fp8(input, w.block_norm_w, norm_q, scales, stats, M, HIDDEN, EPS, stream), "nmt_rmsnorm_quant_fp8");
        ops::gemm_fp8(norm_q, w.in_proj_w, gate, scales, w.in_proj_wscale, M, INTER, HIDDEN, lt, kLtWorkspace, stream);
        ops::gemm_fp8(norm_q, w.in_proj_w + static_cast<size_t>(INTER) * HIDDEN, xbc, scales, w.in_proj_wscale + INTER, M, CONV_DIM,
                      HIDDEN, lt, kLtWorkspace, stream);
        ops::gemm_fp8(norm_q, w.in_proj_w + static_cast<size_t>(INTER + CONV_DIM) * HIDDEN, dt, scales,
                      w.in_proj_wscale + (INTER + CONV_DIM), M, H, HIDDEN, lt, kLtWorkspace, stream);
        ok(nmt_causal_conv1d_silu_split_bf16(xbc, w.conv1d_w, w.conv1d_b, x, Bm, Cm, INTER, GN, GN, conv_state_out, S, B, stream),
           "nmt_causal_conv1d_silu_split_bf16");
        ops::mamba2::ssd_scan_chunked_prefill_bf16<H, P, N, 128>(x, dt, w.A_log, Bm, Cm, w.D, w.dt_bias, y, ssm_state_out, B, S, G,
                                                                 0.f, FLT_MAX, stream);
        ok(nmt_rmsnorm_gated_quant_fp8(y, gate, w.gnorm_w, gnormed, gnorm_q, scales + 1, amax, M, INTER, INTER / G, EPS, stream),
           "nmt_rmsnorm_gated_quant_fp8");
        ops::gemm_fp8(gnorm_q, w.out_proj_w, mixer, scales + 1, w.out_proj_wscale, M, HIDDEN, INTER, lt, kLtWorkspace, stream);
        ops::elementwise_ops_bf16<ops::kElementwiseAdd>(input, mixer, out, rows * HIDDEN, 1.f, nullptr, 0.f, 1.f, stream);
    }
}

template <int HIDDEN, int H, int P, int N, int G, int CONV_K = 4>
inline void mamba_block_decode_fp8(const __nv_bfloat16* input, const Mamba2BlockWeightsFP8& w, float* conv_state,
                                   float* ssm_state, __nv_bfloat16* out, int B, cudaStream_t stream = nullptr) {
    using namespace b200;
    constexpr int INTER = H * P, GN = G * N, CONV_DIM = INTER + 2 * GN, PROJ = INTER + CONV_DIM + H;
    constexpr float EPS = 1e-5f;
    // One sequence per call is what the W8A16 GEMV serves (the reference's gemv_fp8 reads a single activation row too).
    if constexpr (!split_ok(INTER, GN) || CONV_K != 4 || HIDDEN % 64 != 0 || INTER % 64 != 0 || HIDDEN > 10240) {
        return mamba_block_decode_fp8_reference<HIDDEN, H, P, N, G, CONV_K>(input, w, conv_state, ssm_state, out, B, stream);
    } else {
        if (B != 1) return mamba_block_decode_fp8_reference<HIDDEN, H, P, N, G, CONV_K>(input, w, conv_state, ssm_state, out, B, stream);
        // gate | xBC | dt are consecutive rows of in_proj (model/mamba_block.cuh:476-481): one GEMV writes all three.
        bf16* proj = scratch<bf16>(PROJ);
        bf16 *gate = proj, *dt = proj + INTER + CONV_DIM;
        bf16* x = scratch<bf16>(INTER);
        bf16* Bm = scratch<bf16>(GN);
        bf16* Cm = scratch<bf16>(GN);
        bf16* y = scratch<bf16>(INTER);
        // the xBC rows of the projection go through the conv step inside the GEMV's epilogue and land in x | B | C
        ok(nmt_gemv_w8a16_fused_conv_step(input, w.block_norm_w, EPS, w.in_proj_w, w.in_proj_wscale, proj, PROJ, HIDDEN, INTER,
                                          w.conv1d_w, w.conv1d_b, conv_state, x, Bm, Cm, INTER, GN, GN, stream),
           "nmt_gemv_w8a16_fused_conv_step(norm, in_proj, conv step)");
        ok(nmt_ssm_decode_step_bf16(x, dt, w.A_log, Bm, Cm, w.D, w.dt_bias, ssm_state, y, 1, H, P, N, G, 0.f, FLT_MAX, stream),
           "nmt_ssm_decode_step_bf16");
        if constexpr (INTER <= 10240 && (INTER / G) % 8 == 0 && INTER / G <= 2048) {
            ok(nmt_gemv_w8a16_gated(y, gate, w.gnorm_w, EPS, INTER / G, w.out_proj_w, w.out_proj_wscale, input, out, HIDDEN, INTER,
                                    stream), "nmt_gemv_w8a16_gated(gated norm, out_proj, residual)");
        } else {
            bf16* gnormed = scratch<bf16>(INTER);
            ops::rmsnorm_gated_bf16<G>(y, gnormed, w.gnorm_w, gate, 1, INTER, INTER / G, EPS, stream);
            ok(nmt_gemv_w8a16_fused(gnormed, nullptr, 0.f, w.out_proj_w, w.out_proj_wscale, 0, input, out, HIDDEN, INTER, stream),
               "nmt_gemv_w8a16_fused(out_proj, residual)");
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Attention, FP8 weights.  Only the steps around the projections change; the transposes, the SDPA kernels and the KV
// cache writes are the reference's (model/attention_block.cuh:44-95, ops/attention/*).
// ---------------------------------------------------------------------------------------------------------------
template <int HIDDEN, int H_Q, int H_KV, int HEAD = 128>
inline void attention_block_forward_fp8(const __nv_bfloat16* input, const AttnBlockWeightsFP8& w, __nv_bfloat16* out, int S,
                                        __nv_bfloat16* k_cache = nullptr, __nv_bfloat16* v_cache = nullptr, int cache_cap = 0,
                                        cudaStream_t stream = nullptr) {
    using namespace b200;
    namespace att = nemotron::ops::attention;
    constexpr int QD = H_Q * HEAD, KD = H_KV * HEAD;
    constexpr float EPS = 1e-5f;
    if (S <= 0) return;
    if (cache_cap <= 0) cache_cap = S;
    const size_t rows = static_cast<size_t>(S);
    fp8* norm_q = scratch<fp8>(rows * HIDDEN);
    bf16* q = scratch<bf16>(rows * QD);
    bf16* k = scratch<bf16>(rows * KD);
    bf16* v = scratch<bf16>(rows * KD);
    bf16* qt = scratch<bf16>(rows * QD);
    bf16* kt = scratch<bf16>(rows * KD);
    bf16* vt = scratch<bf16>(rows * KD);
    bf16* ot = scratch<bf16>(rows * QD);
    bf16* o = scratch<bf16>(rows * QD);
    fp8* o_q = scratch<fp8>(rows * QD);
    bf16* attn = scratch<bf16>(rows * HIDDEN);
    float* scales = scratch<float>(2);
    unsigned int* amax = scratch<unsigned int>(1);
    char* stats = scratch<char>(nmt_fp8_workspace_bytes(S));
    char* lt = scratch<char>(static_cast<int64_t>(kLtWorkspace));
    ok(nmt_rmsnorm_quant_fp8(input, w.block_norm_w, norm_q, scales, stats, S, HIDDEN, EPS, stream), "nmt_rmsnorm_quant_fp8");
    ops::gemm_fp8(norm_q, w.q_proj_w, q, scales, w.q_proj_wscale, S, QD, HIDDEN, lt, kLtWorkspace, stream);
    ops::gemm_fp8(norm_q, w.k_proj_w, k, scales, w.k_proj_wscale, S, KD, HIDDEN, lt, kLtWorkspace, stream);
    ops::gemm_fp8(norm_q, w.v_proj_w, v, scales, w.v_proj_wscale, S, KD, HIDDEN, lt, kLtWorkspace, stream);
    attn_transpose_shd_to_hsd_launch<bf16>(q, qt, S, H_Q, HEAD, stream);
    attn_transpose_shd_to_hsd_launch<bf16>(k, kt, S, H_KV, HEAD, stream);
    attn_transpose_shd_to_hsd_launch<bf16>(v, vt, S, H_KV, HEAD, stream);
    att::sdpa_prefill_bf16<32, HEAD>(qt, kt, vt, ot, S, H_Q, H_KV, stream);
    attn_transpose_hsd_to_shd_launch<bf16>(ot, o, S, H_Q, HEAD, stream);
    ops::quantize_activation_fp8(o, o_q, scales + 1, amax, rows * QD, stream);       // this library's quantiser (replaced above)
    ops::gemm_fp8(o_q, w.o_proj_w, attn, scales + 1, w.o_proj_wscale, S, HIDDEN, QD, lt, kLtWorkspace, stream);
    ops::elementwise_ops_bf16<ops::kElementwiseAdd>(input, attn, out, rows * HIDDEN, 1.f, nullptr, 0.f, 1.f, stream);
    if (k_cache && v_cache) {                                      // [H_KV, cache_cap, HEAD] caches take the first S positions
        const size_t row_bytes = static_cast<size_t>(S) * HEAD * sizeof(bf16), pitch = static_cast<size_t>(cache_cap) * HEAD * sizeof(bf16);
        cudaMemcpy2DAsync(k_cache, pitch, kt, row_bytes, row_bytes, H_KV, cudaMemcpyDeviceToDevice, stream);
        cudaMemcpy2DAsync(v_cache, pitch, vt, row_bytes, row_bytes, H_KV, cudaMemcpyDeviceToDevice, stream);
    }
}

template <int HIDDEN, int H_Q, int H_KV, int HEAD = 128>
inline void attention_block_decode_fp8(const __nv_bfloat16* input, const AttnBlockWeightsFP8& w, __nv_bfloat16* k_cache,
                                       __nv_bfloat16* v_cache, int S_cache, int cache_cap, __nv_bfloat16* out,
                                       cudaStream_t stream = nullptr) {
    using namespace b200;
    namespace att = nemotron::ops::attention;
    constexpr int QD = H_Q * HEAD, KD = H_KV * HEAD;
    constexpr float EPS = 1e-5f;
    if constexpr (HIDDEN % 64 != 0 || QD % 64 != 0 || HIDDEN > 10240) {
        return attention_block_decode_fp8_reference<HIDDEN, H_Q, H_KV, HEAD>(input, w, k_cache, v_cache, S_cache, cache_cap, out, stream);
    } else {
        bf16* q = scratch<bf16>(QD);
        bf16* knew = scratch<bf16>(KD);
        bf16* vnew = scratch<bf16>(KD);
        bf16* ot = scratch<bf16>(QD);
        // q, k and v are three matrices, so three GEMVs; each normalises its own copy of the token (a 3136-wide row), which
        // is cheaper than a launch of its own for the norm
        ok(nmt_gemv_w8a16_fused(input, w.block_norm_w, EPS, w.q_proj_w, w.q_proj_wscale, 0, nullptr, q, QD, HIDDEN, stream), "nmt_gemv_w8a16_fused(norm, q_proj)");
        ok(nmt_gemv_w8a16_fused(input, w.block_norm_w, EPS, w.k_proj_w, w.k_proj_wscale, 0, nullptr, knew, KD, HIDDEN, stream), "nmt_gemv_w8a16_fused(norm, k_proj)");
        ok(nmt_gemv_w8a16_fused(input, w.block_norm_w, EPS, w.v_proj_w, w.v_proj_wscale, 0, nullptr, vnew, KD, HIDDEN, stream), "nmt_gemv_w8a16_fused(norm, v_proj)");
        att::sdpa_decode_bf16<HEAD>(q, k_cache, v_cache, ot, knew, vnew, S_cache, cache_cap, H_Q, H_KV, stream);
        ok(nmt_gemv_w8a16_fused(ot, nullptr, 0.f, w.o_proj_w, w.o_proj_wscale, 0, input, out, HIDDEN, QD, stream), "nmt_gemv_w8a16_fused(o_proj, residual)");
    }
}

}  // namespace nemotron::model

#endif  // NEMOTRON_B200_SHIM_BLOCKS_CUH
