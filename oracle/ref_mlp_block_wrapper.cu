// TEST INFRASTRUCTURE — extern "C" doors onto the reference's OWN MLP block (model/mlp_block.cuh),
// compiled from its headers in place.  The Makefile builds this file twice:
//   libref_mlp_stock.so  with the reference's include directory only  -> the reference's kernels
//   libref_mlp_shim.so   with include/nemotron_b200_shim first        -> the same block code, unchanged,
//                        running its RMSNorm / relu^2 / residual add on libnemotron_b200.so
// so a test can show that the block output is the same through the drop-in.
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include "tensor/tensor.h"
#include "tensor/allocator.cuh"
#include "model/mlp_block.cuh"

using namespace nemotron;
using namespace nemotron::model;
using bf16 = __nv_bfloat16;

#define BLK_API extern "C" __attribute__((visibility("default")))

BLK_API int blk_mlp_forward_fp32(const float* in, const float* norm_w, const float* up_w, const float* down_w,
                                 float* out, int M, int hidden, int inter) {
    MLPBlockWeightsFP32 w{norm_w, up_w, down_w};
    if (hidden == 64 && inter == 256) mlp_block_forward_fp32<64, 256>(in, w, out, M, nullptr);
    else return -1;
    return static_cast<int>(cudaGetLastError());
}

BLK_API int blk_mlp_forward_bf16(const void* in, const float* norm_w, const void* up_w, const void* down_w,
                                 void* out, int M, int hidden, int inter) {
    MLPBlockWeightsBF16 w{norm_w, static_cast<const bf16*>(up_w), static_cast<const bf16*>(down_w)};
    auto I = static_cast<const bf16*>(in);
    auto O = static_cast<bf16*>(out);
    if (hidden == 64 && inter == 256) mlp_block_forward_bf16<64, 256>(I, w, O, M, nullptr);
    else if (hidden == 3136 && inter == 12544) mlp_block_forward_bf16<3136, 12544>(I, w, O, M, nullptr);
    else return -1;
    return static_cast<int>(cudaGetLastError());
}

// The reference's own activation quantiser (ops/gemm.cuh:291-307), for bit-level comparison.
BLK_API int blk_quantize_activation_fp8(const void* x, void* out, float* scale, unsigned int* amax, size_t n) {
    nemotron::ops::quantize_activation_fp8(static_cast<const bf16*>(x), static_cast<__nv_fp8_e4m3*>(out), scale, amax, n, nullptr);
    return static_cast<int>(cudaGetLastError());
}

// The block's workspaces come from the reference's bump allocator; callers rewind it between calls
// exactly as engine.py does through binding.reset_allocator() (binding.cu:59).
BLK_API void blk_reset_allocator() { default_allocator().rewind(); }
BLK_API void blk_free_allocator() { default_allocator().reset(); }
BLK_API int blk_set_device(int d) { return static_cast<int>(cudaSetDevice(d)); }
