// Source-level drop-in for the reference header ops/embedding.cuh (see reduce.cuh in this directory).
// embedding_lookup<Hidden>(table, int64 ids, out, num_tokens, stream) as in ops/embedding.cuh:53-66.  Like the
// reference it does not range-check the ids; use nmt_embedding_bf16_i64 directly to get the checked form.
#ifndef NEMOTRON_B200_SHIM_EMBEDDING_CUH
#define NEMOTRON_B200_SHIM_EMBEDDING_CUH
// The reference's own guard: wherever its header of the same name is included later (binding.cu includes it by a path
// relative to itself), it is skipped, so the launchers below are the only definitions.
#ifndef NEMOTRON_INFER_EMBEDDING_CUH
#define NEMOTRON_INFER_EMBEDDING_CUH
#endif

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstddef>
#include <cstdint>

#include "../../nemotron_b200.h"
#include "nmt_shim_check.h"

namespace nemotron::ops {

template <int Hidden>
inline void embedding_lookup(const __nv_bfloat16* table, const int64_t* token_ids, __nv_bfloat16* out,
                             const size_t num_tokens, cudaStream_t stream = nullptr) {
    static_assert(Hidden % 8 == 0, "rows are copied in 16-byte units");
    detail::nmt_shim_check(nmt_embedding_bf16_i64(table, token_ids, out, static_cast<int64_t>(num_tokens), Hidden, 0, nullptr, stream), "nmt_embedding_bf16_i64");
}

}  // namespace nemotron::ops

#endif  // NEMOTRON_B200_SHIM_EMBEDDING_CUH
