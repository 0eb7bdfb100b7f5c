// TEST INFRASTRUCTURE — extern "C" doors onto the reference's OWN Mamba-2 block (model/mamba_block.cuh) at the
// tiny configuration of its golden emitter (tools/dump_mamba_block.py: HIDDEN 64, H 4, P 16, N 16, G 2, K 4).
// Built twice by the Makefile, like the MLP block: on the reference's kernels ("stock") and, unchanged, on
// include/nemotron_b200_shim + libnemotron_b200.so ("shim"), where its RMSNorm, gated RMSNorm and residual add
// run on this library.
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include "tensor/tensor.h"
#include "tensor/allocator.cuh"
#include "model/mamba_block.cuh"

using namespace nemotron;
using namespace nemotron::model;
using bf16 = __nv_bfloat16;

#define BLK_API extern "C" __attribute__((visibility("default")))

BLK_API int blk_mamba_forward_fp32(const float* in, const float* norm_w, const float* in_proj, const float* conv_w,
                                   const float* conv_b, const float* A_log, const float* D, const float* dt_bias,
                                   const float* gnorm_w, const float* out_proj, float* out, int B, int S) {
    Mamba2BlockWeightsFP32 w{norm_w, in_proj, conv_w, conv_b, A_log, D, dt_bias, gnorm_w, out_proj};
    mamba_block_forward_fp32<64, 4, 16, 16, 2, 4>(in, w, out, B, S, nullptr);
    return static_cast<int>(cudaGetLastError());
}

BLK_API int blk_mamba_forward_bf16(const void* in, const float* norm_w, const void* in_proj, const float* conv_w,
                                   const float* conv_b, const float* A_log, const float* D, const float* dt_bias,
                                   const float* gnorm_w, const void* out_proj, void* out, int B, int S) {
    Mamba2BlockWeightsBF16 w{norm_w, static_cast<const bf16*>(in_proj), conv_w, conv_b, A_log, D, dt_bias, gnorm_w,
                             static_cast<const bf16*>(out_proj)};
    mamba_block_forward_bf16<64, 4, 16, 16, 2, 4>(static_cast<const bf16*>(in), w, static_cast<bf16*>(out), B, S,
                                                  nullptr, nullptr, nullptr);
    return static_cast<int>(cudaGetLastError());
}

BLK_API void blk_reset_allocator() { default_allocator().rewind(); }
BLK_API void blk_free_allocator() { default_allocator().reset(); }
BLK_API int blk_set_device(int d) { return static_cast<int>(cudaSetDevice(d)); }
