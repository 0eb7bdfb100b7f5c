// TEST INFRASTRUCTURE — extern "C" doors onto the reference's OWN host launchers,
// compiled from the reference's headers where they lie (nothing is copied): the
// Makefile passes -I <reference>/nemotron_infer/csrc/include.  The resulting
// library is used by the GPU parity tests as a second checker and by bench.py to
// time "the reference kernels recompiled for sm_100a" beside the new kernels.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cfloat>
#include <cstdint>

#include "tensor/tensor.h"
#include "ops/reduce.cuh"        // rmsnorm_{fp32,bf16}, rmsnorm_gated_{fp32,bf16}<Group>
#include "ops/elementwise.cuh"   // elementwise_ops_{fp32,bf16}<Op>
#include "ops/embedding.cuh"     // embedding_lookup<Hidden>
#include "ops/gemv.cuh"                   // gemv_fp8
#include "ops/mamba2/causal_conv1d.cuh"   // causal_conv1d_prefill_{fp32,bf16}
#include "ops/mamba2/ssm.cuh"             // ssm_decode_bf16<H, D, N>
#include "ops/attention/sdpa_decode.cuh"  // sdpa_decode_bf16<HEAD>

using namespace nemotron::ops;
using bf16 = __nv_bfloat16;

#define REF_API extern "C" __attribute__((visibility("default")))

static int last() { return static_cast<int>(cudaGetLastError()); }

REF_API int ref_rmsnorm_fp32(const float* x, float* y, const float* w, size_t rows, size_t cols, float eps, void* st) {
    rmsnorm_fp32(x, y, w, rows, cols, eps, static_cast<cudaStream_t>(st));
    return last();
}
REF_API int ref_rmsnorm_bf16(const void* x, void* y, const float* w, size_t rows, size_t cols, float eps, void* st) {
    rmsnorm_bf16(static_cast<const bf16*>(x), static_cast<bf16*>(y), w, rows, cols, eps, static_cast<cudaStream_t>(st));
    return last();
}

template <int G>
static void gated_bf16(const void* y, void* out, const float* w, const void* z, size_t rows, size_t cols, size_t gs,
                       float eps, cudaStream_t st) {
    rmsnorm_gated_bf16<G>(static_cast<const bf16*>(y), static_cast<bf16*>(out), w, static_cast<const bf16*>(z),
                          rows, cols, gs, eps, st);
}
// Group is a template parameter in the reference (binding.cu uses G = 8); the door covers the counts the tests use.
REF_API int ref_rmsnorm_gated_bf16(const void* y, const void* z, const float* w, void* out, size_t rows, size_t cols,
                                   size_t gs, float eps, void* stv) {
    cudaStream_t st = static_cast<cudaStream_t>(stv);
    switch (cols / gs) {
        case 1: gated_bf16<1>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 2: gated_bf16<2>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 3: gated_bf16<3>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 4: gated_bf16<4>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 8: gated_bf16<8>(y, out, w, z, rows, cols, gs, eps, st); break;
        default: return -1;
    }
    return last();
}
REF_API int ref_rmsnorm_gated_fp32(const float* y, const float* z, const float* w, float* out, size_t rows, size_t cols,
                                   size_t gs, float eps, void* stv) {
    cudaStream_t st = static_cast<cudaStream_t>(stv);
    switch (cols / gs) {
        case 1: rmsnorm_gated_fp32<1>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 2: rmsnorm_gated_fp32<2>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 3: rmsnorm_gated_fp32<3>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 4: rmsnorm_gated_fp32<4>(y, out, w, z, rows, cols, gs, eps, st); break;
        case 8: rmsnorm_gated_fp32<8>(y, out, w, z, rows, cols, gs, eps, st); break;
        default: return -1;
    }
    return last();
}

REF_API int ref_add_bf16(const void* a, const void* b, void* out, size_t n, void* st) {
    elementwise_ops_bf16<kElementwiseAdd>(static_cast<const bf16*>(a), static_cast<const bf16*>(b),
                                          static_cast<bf16*>(out), n, 1.f, nullptr, 0.f, 1.f,
                                          static_cast<cudaStream_t>(st));
    return last();
}
REF_API int ref_relu2_bf16(const void* u, void* out, size_t n, void* st) {
    // Same call shape as model/mlp_block.cuh:100 (in1 = in0).
    elementwise_ops_bf16<kElementwiseRelu2>(static_cast<const bf16*>(u), static_cast<const bf16*>(u),
                                            static_cast<bf16*>(out), n, 1.f, nullptr, 0.f, 1.f,
                                            static_cast<cudaStream_t>(st));
    return last();
}
REF_API int ref_add_fp32(float* a, float* b, float* out, size_t n, void* st) {
    elementwise_ops_fp32<kElementwiseAdd>(a, b, out, n, 1.f, nullptr, 0.f, 1.f, static_cast<cudaStream_t>(st));
    return last();
}
REF_API int ref_relu2_fp32(float* u, float* out, size_t n, void* st) {
    elementwise_ops_fp32<kElementwiseRelu2>(u, u, out, n, 1.f, nullptr, 0.f, 1.f, static_cast<cudaStream_t>(st));
    return last();
}

// Hidden is a template parameter in the reference (binding.cu uses 3136; its tests also use 128).
REF_API int ref_embedding_i64(const void* table, const int64_t* ids, void* out, size_t num_tokens, int hidden, void* stv) {
    cudaStream_t st = static_cast<cudaStream_t>(stv);
    auto T = static_cast<const bf16*>(table);
    auto O = static_cast<bf16*>(out);
    switch (hidden) {
        case 128: embedding_lookup<128>(T, ids, O, num_tokens, st); break;
        case 3136: embedding_lookup<3136>(T, ids, O, num_tokens, st); break;
        default: return -1;
    }
    return last();
}

REF_API int ref_causal_conv1d_bf16(const void* x, const float* w, const float* b, void* y, float* state_out, int conv_dim,
                                   int S, int batch, void* st) {
    mamba2::causal_conv1d_prefill_bf16<64>(static_cast<const bf16*>(x), w, b, static_cast<bf16*>(y), state_out, conv_dim, S,
                                           batch, static_cast<cudaStream_t>(st));
    return last();
}

REF_API int ref_gemv_fp8(const void* x, const void* W, const float* w_scale, void* y, int N, int K, void* st) {
    gemv_fp8(static_cast<const bf16*>(x), static_cast<const __nv_fp8_e4m3*>(W), w_scale, static_cast<bf16*>(y), N, K,
             static_cast<cudaStream_t>(st));
    return last();
}

REF_API int ref_set_device(int d) { return static_cast<int>(cudaSetDevice(d)); }

// The single-token SSM step at the model's dimensions and at those of the reference's dump script, launched as the
// decode blocks launch it (model/mamba_block.cuh:298-301).
REF_API int ref_ssm_decode_bf16(const void* x, const void* dt, const float* A_log, const void* B, const void* C, const float* D,
                                const float* dt_bias, float* state, void* y, int batch, int H, int P, int N, int groups, void* st) {
    auto X = static_cast<const bf16*>(x);
    auto DT = static_cast<const bf16*>(dt);
    auto Bp = static_cast<const bf16*>(B);
    auto Cp = static_cast<const bf16*>(C);
    auto Y = static_cast<bf16*>(y);
    cudaStream_t s = static_cast<cudaStream_t>(st);
    if (H == 96 && P == 80 && N == 128)
        mamba2::ssm_decode_bf16<96, 80, 128><<<dim3(batch * H), 128, 0, s>>>(X, DT, A_log, Bp, Cp, D, state, Y, dt_bias, batch, groups, 0.f, FLT_MAX);
    else if (H == 4 && P == 16 && N == 16)
        mamba2::ssm_decode_bf16<4, 16, 16><<<dim3(batch * H), 128, 0, s>>>(X, DT, A_log, Bp, Cp, D, state, Y, dt_bias, batch, groups, 0.f, FLT_MAX);
    else
        return -1;
    return last();
}

// Decode attention as the attention blocks call it (model/attention_block.cuh:251); its scratch is the reference's own.
REF_API int ref_sdpa_decode_bf16(const void* Q, void* K_cache, void* V_cache, void* O, const void* K_new, const void* V_new,
                                 int S_cache, int total_S, int num_heads, int num_kv_heads, void* st) {
    attention::sdpa_decode_bf16<128>(static_cast<const bf16*>(Q), static_cast<bf16*>(K_cache), static_cast<bf16*>(V_cache),
                                     static_cast<bf16*>(O), static_cast<const bf16*>(K_new), static_cast<const bf16*>(V_new), S_cache,
                                     total_S, num_heads, num_kv_heads, static_cast<cudaStream_t>(st));
    return last();
}
