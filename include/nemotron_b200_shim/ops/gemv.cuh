// Source-level drop-in for the reference header ops/gemv.cuh (see reduce.cuh in this directory for how the
// drop-in headers are used).  gemv_fp8(x, W, w_scale, y, N, K, stream) as in ops/gemv.cuh:92-104 - the W8A16
// product of the single-token decode projections - forwarded to nmt_gemv_w8a16.  W and w_scale are model
// constants to that kernel (see its ordering contract in nemotron_b200.h).
#ifndef NEMOTRON_B200_SHIM_GEMV_CUH
#define NEMOTRON_B200_SHIM_GEMV_CUH
#ifndef NEMOTRON_INFER_OPS_GEMV_CUH
#define NEMOTRON_INFER_OPS_GEMV_CUH      // the reference's own guard: its header is skipped wherever it is included later
#endif

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>

#include "../../nemotron_b200.h"
#include "nmt_shim_check.h"

namespace nemotron::ops {

inline void gemv_fp8(const __nv_bfloat16* x, const __nv_fp8_e4m3* W, const float* w_scale, __nv_bfloat16* y, int N,
                     int K, cudaStream_t stream = nullptr) {
    detail::nmt_shim_check(nmt_gemv_w8a16(x, W, w_scale, y, static_cast<int64_t>(N), static_cast<int64_t>(K), stream),
                           "nmt_gemv_w8a16");
}

}  // namespace nemotron::ops

#endif  // NEMOTRON_B200_SHIM_GEMV_CUH
