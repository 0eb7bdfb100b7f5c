// TEST INFRASTRUCTURE - extern "C" doors onto the reference's OWN blocks (model/{mlp,mamba,attention}_block.cuh),
// compiled from its headers in place at the tiny configurations of its golden emitters (tools/dump_*.py) and, for
// the MLP, at model width.  One file, one bump allocator for all blocks (as in the reference's binding.cu), so that
// a stack of blocks behaves as it does under engine.py.  The Makefile builds it three times:
//   libref_blocks_stock.so   the reference's include directory only              -> the reference's kernels
//   libref_blocks_shim.so    include/nemotron_b200_shim first                    -> the same block code, unchanged, with its
//                            norms / relu^2 / adds / W8A16 GEMVs on libnemotron_b200.so
//   libref_blocks_fused.so   model/blocks_b200.cuh pre-included                  -> the fused block forms under the
//                            reference's names (and its quantiser replaced)
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "tensor/tensor.h"
#include "tensor/allocator.cuh"
#include "model/mlp_block.cuh"
#include "model/mamba_block.cuh"
#include "model/attention_block.cuh"

using namespace nemotron;
using namespace nemotron::model;
using bf16 = __nv_bfloat16;
using fp8 = __nv_fp8_e4m3;

#define BLK_API extern "C" __attribute__((visibility("default")))
static int last_error() { return static_cast<int>(cudaGetLastError()); }

// ---- MLP ------------------------------------------------------------------------------------------------------
BLK_API int blk_mlp_forward_fp32(const float* in, const float* norm_w, const float* up_w, const float* down_w,
                                 float* out, int M, int hidden, int inter) {
    MLPBlockWeightsFP32 w{norm_w, up_w, down_w};
    if (hidden == 64 && inter == 256) mlp_block_forward_fp32<64, 256>(in, w, out, M, nullptr);
    else return -1;
    return last_error();
}

BLK_API int blk_mlp_forward_bf16(const void* in, const float* norm_w, const void* up_w, const void* down_w,
                                 void* out, int M, int hidden, int inter) {
    MLPBlockWeightsBF16 w{norm_w, static_cast<const bf16*>(up_w), static_cast<const bf16*>(down_w)};
    auto I = static_cast<const bf16*>(in);
    auto O = static_cast<bf16*>(out);
    if (hidden == 64 && inter == 256) mlp_block_forward_bf16<64, 256>(I, w, O, M, nullptr);
    else if (hidden == 256 && inter == 512) mlp_block_forward_bf16<256, 512>(I, w, O, M, nullptr);
    else if (hidden == 3136 && inter == 12544) mlp_block_forward_bf16<3136, 12544>(I, w, O, M, nullptr);
    else return -1;
    return last_error();
}

BLK_API int blk_mlp_forward_fp8(const void* in, const float* norm_w, const void* up_w, const float* up_s,
                                const void* down_w, const float* down_s, void* out, int M, int hidden, int inter) {
    MLPBlockWeightsFP8 w{norm_w, static_cast<const fp8*>(up_w), up_s, static_cast<const fp8*>(down_w), down_s};
    auto I = static_cast<const bf16*>(in);
    auto O = static_cast<bf16*>(out);
    if (hidden == 64 && inter == 256) mlp_block_forward_fp8<64, 256>(I, w, O, M, nullptr);
    else if (hidden == 3136 && inter == 12544) mlp_block_forward_fp8<3136, 12544>(I, w, O, M, nullptr);
    else return -1;
    return last_error();
}

// ---- Mamba-2 at the emitter's configuration (HIDDEN 64, H 4, P 16, N 16, G 2, K 4) ---------------------------------
#define MAMBA_CFG 64, 4, 16, 16, 2, 4
BLK_API int blk_mamba_forward_fp32(const float* in, const float* norm_w, const float* in_proj, const float* conv_w,
                                   const float* conv_b, const float* A_log, const float* D, const float* dt_bias,
                                   const float* gnorm_w, const float* out_proj, float* out, int B, int S) {
    Mamba2BlockWeightsFP32 w{norm_w, in_proj, conv_w, conv_b, A_log, D, dt_bias, gnorm_w, out_proj};
    mamba_block_forward_fp32<MAMBA_CFG>(in, w, out, B, S, nullptr);
    return last_error();
}

BLK_API int blk_mamba_forward_bf16(const void* in, const float* norm_w, const void* in_proj, const float* conv_w,
                                   const float* conv_b, const float* A_log, const float* D, const float* dt_bias,
                                   const float* gnorm_w, const void* out_proj, void* out, int B, int S,
                                   float* conv_state_out, float* ssm_state_out) {
    Mamba2BlockWeightsBF16 w{norm_w, static_cast<const bf16*>(in_proj), conv_w, conv_b, A_log, D, dt_bias, gnorm_w,
                             static_cast<const bf16*>(out_proj)};
    mamba_block_forward_bf16<MAMBA_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(out), B, S, conv_state_out,
                                        ssm_state_out, nullptr);
    return last_error();
}

BLK_API int blk_mamba_decode_bf16(const void* in, const float* norm_w, const void* in_proj, const float* conv_w,
                                  const float* conv_b, const float* A_log, const float* D, const float* dt_bias,
                                  const float* gnorm_w, const void* out_proj, float* conv_state, float* ssm_state,
                                  void* out, int B) {
    Mamba2BlockWeightsBF16 w{norm_w, static_cast<const bf16*>(in_proj), conv_w, conv_b, A_log, D, dt_bias, gnorm_w,
                             static_cast<const bf16*>(out_proj)};
    mamba_block_decode_bf16<MAMBA_CFG>(static_cast<const bf16*>(in), w, conv_state, ssm_state, static_cast<bf16*>(out), B, nullptr);
    return last_error();
}

BLK_API int blk_mamba_forward_fp8(const void* in, const float* norm_w, const void* in_proj, const float* in_proj_s,
                                  const float* conv_w, const float* conv_b, const float* A_log, const float* D,
                                  const float* dt_bias, const float* gnorm_w, const void* out_proj, const float* out_proj_s,
                                  void* out, int B, int S, float* conv_state_out, float* ssm_state_out) {
    Mamba2BlockWeightsFP8 w{norm_w, static_cast<const fp8*>(in_proj), in_proj_s, conv_w, conv_b, A_log, D, dt_bias, gnorm_w,
                            static_cast<const fp8*>(out_proj), out_proj_s};
    mamba_block_forward_fp8<MAMBA_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(out), B, S, conv_state_out,
                                       ssm_state_out, nullptr);
    return last_error();
}

BLK_API int blk_mamba_decode_fp8(const void* in, const float* norm_w, const void* in_proj, const float* in_proj_s,
                                 const float* conv_w, const float* conv_b, const float* A_log, const float* D,
                                 const float* dt_bias, const float* gnorm_w, const void* out_proj, const float* out_proj_s,
                                 float* conv_state, float* ssm_state, void* out, int B) {
    Mamba2BlockWeightsFP8 w{norm_w, static_cast<const fp8*>(in_proj), in_proj_s, conv_w, conv_b, A_log, D, dt_bias, gnorm_w,
                            static_cast<const fp8*>(out_proj), out_proj_s};
    mamba_block_decode_fp8<MAMBA_CFG>(static_cast<const bf16*>(in), w, conv_state, ssm_state, static_cast<bf16*>(out), B, nullptr);
    return last_error();
}

// ---- attention at the emitter's configuration (HIDDEN 256, 4 query heads, 2 KV heads, head 128) -------------------
#define ATTN_CFG 256, 4, 2, 128
BLK_API int blk_attn_forward_fp32(const float* in, const float* norm_w, const float* q_w, const float* k_w, const float* v_w,
                                  const float* o_w, float* out, int S) {
    AttnBlockWeightsFP32 w{norm_w, q_w, k_w, v_w, o_w};
    attention_block_forward_fp32<ATTN_CFG>(in, w, out, S, nullptr);
    return last_error();
}

BLK_API int blk_attn_forward_bf16(const void* in, const float* norm_w, const void* q_w, const void* k_w, const void* v_w,
                                  const void* o_w, void* out, int S, void* k_cache, void* v_cache, int cache_cap) {
    AttnBlockWeightsBF16 w{norm_w, static_cast<const bf16*>(q_w), static_cast<const bf16*>(k_w), static_cast<const bf16*>(v_w),
                           static_cast<const bf16*>(o_w)};
    attention_block_forward_bf16<ATTN_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(out), S,
                                           static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), cache_cap, nullptr);
    return last_error();
}

BLK_API int blk_attn_decode_bf16(const void* in, const float* norm_w, const void* q_w, const void* k_w, const void* v_w,
                                 const void* o_w, void* k_cache, void* v_cache, int S_cache, int cache_cap, void* out) {
    AttnBlockWeightsBF16 w{norm_w, static_cast<const bf16*>(q_w), static_cast<const bf16*>(k_w), static_cast<const bf16*>(v_w),
                           static_cast<const bf16*>(o_w)};
    attention_block_decode_bf16<ATTN_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache),
                                          S_cache, cache_cap, static_cast<bf16*>(out), nullptr);
    return last_error();
}

BLK_API int blk_attn_forward_fp8(const void* in, const float* norm_w, const void* q_w, const float* q_s, const void* k_w,
                                 const float* k_s, const void* v_w, const float* v_s, const void* o_w, const float* o_s, void* out,
                                 int S, void* k_cache, void* v_cache, int cache_cap) {
    AttnBlockWeightsFP8 w{norm_w, static_cast<const fp8*>(q_w), q_s, static_cast<const fp8*>(k_w), k_s, static_cast<const fp8*>(v_w), v_s,
                          static_cast<const fp8*>(o_w), o_s};
    attention_block_forward_fp8<ATTN_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(out), S, static_cast<bf16*>(k_cache),
                                          static_cast<bf16*>(v_cache), cache_cap, nullptr);
    return last_error();
}

BLK_API int blk_attn_decode_fp8(const void* in, const float* norm_w, const void* q_w, const float* q_s, const void* k_w,
                                const float* k_s, const void* v_w, const float* v_s, const void* o_w, const float* o_s,
                                void* k_cache, void* v_cache, int S_cache, int cache_cap, void* out) {
    AttnBlockWeightsFP8 w{norm_w, static_cast<const fp8*>(q_w), q_s, static_cast<const fp8*>(k_w), k_s, static_cast<const fp8*>(v_w), v_s,
                          static_cast<const fp8*>(o_w), o_s};
    attention_block_decode_fp8<ATTN_CFG>(static_cast<const bf16*>(in), w, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), S_cache,
                                         cache_cap, static_cast<bf16*>(out), nullptr);
    return last_error();
}

// The activation quantiser the blocks call (ops/gemm.cuh:291-307; this library's in the fused build).
BLK_API int blk_quantize_activation_fp8(const void* x, void* out, float* scale, unsigned int* amax, size_t n) {
    nemotron::ops::quantize_activation_fp8(static_cast<const bf16*>(x), static_cast<fp8*>(out), scale, amax, n, nullptr);
    return last_error();
}

// The block's workspaces come from the reference's bump allocator; callers rewind it between blocks exactly as
// engine.py does through binding.reset_allocator() (binding.cu:59, engine.py:263).
BLK_API void blk_reset_allocator() { default_allocator().rewind(); }
BLK_API void blk_free_allocator() { default_allocator().reset(); }
BLK_API int blk_set_device(int d) { return static_cast<int>(cudaSetDevice(d)); }
