// Status handling shared by the drop-in headers in this directory.
//
// The reference launchers return void and check nothing (ops/reduce.cuh:229-244); the library behind these
// headers validates every call and launches NOTHING when it rejects one (a weight vector that is not 16-byte
// aligned, `out` aliasing an input of the fused add + norm, a launch the CUDA runtime refused ...).  Dropping
// that status would leave the output buffer stale with no sign of it, so a rejected call ends the process the
// way the reference's own TENSOR_CHECK does (tensor/allocator.cuh:25-30): one line on stderr, then abort().
#ifndef NEMOTRON_B200_SHIM_CHECK_H
#define NEMOTRON_B200_SHIM_CHECK_H

#include <cstdio>
#include <cstdlib>

#include "../../nemotron_b200.h"

namespace nemotron::ops::detail {

inline void nmt_shim_check(int status, const char* what) {
    if (status == NMT_OK) return;
    std::fprintf(stderr, "[FATAL] nemotron_b200 shim: %s rejected: %s%s%s\n", what, nmt_status_string(status),
                 status == NMT_ERR_LAUNCH ? ": " : "", status == NMT_ERR_LAUNCH ? nmt_last_cuda_error() : "");
    std::abort();
}

}  // namespace nemotron::ops::detail

#endif  // NEMOTRON_B200_SHIM_CHECK_H
