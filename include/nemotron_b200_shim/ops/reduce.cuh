// Source-level drop-in for the reference header ops/reduce.cuh.
//
// Put  -I <this repo>/include/nemotron_b200_shim  BEFORE the reference's own include directory and the
// reference's block code (model/mlp_block.cuh, model/mamba_block.cuh, model/attention_block.cuh, binding.cu)
// compiles unchanged: `#include "ops/reduce.cuh"` resolves here, and the host launchers below keep the
// reference's names, template parameters, argument order and defaults (ops/reduce.cuh:113-128, 229-244,
// 360-377, 510-527) while forwarding to libnemotron_b200.so.  Like the originals they return void and launch
// asynchronously on `stream`; a call the library rejects (nothing launched) aborts the process with a message,
// see nmt_shim_check.h.
#ifndef NEMOTRON_B200_SHIM_REDUCE_CUH
#define NEMOTRON_B200_SHIM_REDUCE_CUH
// The reference's own guard: wherever its header of the same name is included later (binding.cu includes it by a path
// relative to itself), it is skipped, so the launchers below are the only definitions.
#ifndef NEMOTRON_INFER_REDUCE_CUH
#define NEMOTRON_INFER_REDUCE_CUH
#endif

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstddef>

#include "../../nemotron_b200.h"
#include "nmt_shim_check.h"

namespace nemotron::ops {

inline void rmsnorm_fp32(const float* in0, float* out0, const float* weight, const size_t rows, const size_t cols,
                         const float eps = 1e-5f, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_rmsnorm_f32(in0, out0, weight, static_cast<int64_t>(rows), static_cast<int64_t>(cols), eps, stream), "nmt_rmsnorm_f32");
}

inline void rmsnorm_bf16(const __nv_bfloat16* in0, __nv_bfloat16* out0, const float* weight, const size_t rows,
                         const size_t cols, const float eps = 1e-5f, cudaStream_t stream = nullptr) {
    // every rmsnorm_bf16 of the reference opens a block (or is the final norm): the head entry point runs the plain
    // kernel unless the previous block's fused tail already produced exactly this tensor (see nmt_fuse_next_norm)
    detail::nmt_shim_check(nmt_block_head_rmsnorm_bf16(in0, out0, weight, static_cast<int64_t>(rows), static_cast<int64_t>(cols), eps, stream), "nmt_block_head_rmsnorm_bf16");
}

// Group stays a template parameter for source compatibility; the library takes the group size at run time.
template <int Group>
inline void rmsnorm_gated_fp32(const float* in0, float* out0, const float* weight, const float* gate,
                               const size_t rows, const size_t cols, const size_t group_size,
                               const float eps = 1e-5f, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_rmsnorm_gated_f32(in0, gate, weight, out0, static_cast<int64_t>(rows), static_cast<int64_t>(cols),
                          static_cast<int64_t>(group_size), eps, stream), "nmt_rmsnorm_gated_f32");
}

template <int Group>
inline void rmsnorm_gated_bf16(const __nv_bfloat16* in0, __nv_bfloat16* out0, const float* weight,
                               const __nv_bfloat16* gate, const size_t rows, const size_t cols,
                               const size_t group_size, const float eps = 1e-5f, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_rmsnorm_gated_bf16(in0, gate, weight, out0, static_cast<int64_t>(rows), static_cast<int64_t>(cols),
                           static_cast<int64_t>(group_size), eps, stream), "nmt_rmsnorm_gated_bf16");
}

// Not in the reference: the block-tail add fused with the next block's pre-norm (one launch, one HBM pass).
inline void add_rmsnorm_bf16(const __nv_bfloat16* x, const __nv_bfloat16* r, const float* weight,
                             __nv_bfloat16* out_res, __nv_bfloat16* out, const size_t rows, const size_t cols,
                             const float eps = 1e-5f, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_add_rmsnorm_bf16(x, r, weight, out_res, out, static_cast<int64_t>(rows), static_cast<int64_t>(cols), eps, stream), "nmt_add_rmsnorm_bf16");
}

}  // namespace nemotron::ops

#endif  // NEMOTRON_B200_SHIM_REDUCE_CUH
