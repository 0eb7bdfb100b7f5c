// Token-embedding gather: out[i, :] = table[ids[i], :], a bit-exact row copy.
//
// Register variant: one warp owns one token.  A 3136-wide row is 392 16-byte
// vectors = 13 lane slots; all 13 loads are issued before the first store, so a
// warp keeps a whole 6272-byte row in flight.  Ids outside [0, vocab) are never
// dereferenced: the output row is zero-filled and an error flag is raised.
#include "nmt_common.cuh"

namespace nmt {

template <int SLOTS, typename IdT>
__global__ void __launch_bounds__(256)
embedding_rowwarp_kernel(const uint4* __restrict__ table, const IdT* __restrict__ ids, uint4* __restrict__ out,
                         int64_t num_tokens, int nv, int64_t vocab, int32_t* err_flag) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * warps_per_cta;
#pragma unroll 1
    for (int64_t t = warp0; t < num_tokens; t += nwarps) {
        const int64_t id = static_cast<int64_t>(__ldg(ids + t));
        const bool ok = vocab <= 0 || (id >= 0 && id < vocab);
        if (!ok && lane == 0 && err_flag) atomicExch(err_flag, 1);
        const uint4* src = table + (ok ? id : 0) * nv;
        uint4 v[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int i = s * 32 + lane;
            v[s] = (ok && i < nv) ? ld_stream(src + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int i = s * 32 + lane;
            if (i < nv) st_stream(out + t * nv + i, v[s]);
        }
    }
    pdl_trigger();
}

// Any width: one warp per token, looped.
template <typename IdT>
__global__ void __launch_bounds__(256)
embedding_generic_kernel(const uint4* __restrict__ table, const IdT* __restrict__ ids, uint4* __restrict__ out,
                         int64_t num_tokens, int64_t nv, int64_t vocab, int32_t* err_flag) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * warps_per_cta;
#pragma unroll 1
    for (int64_t t = warp0; t < num_tokens; t += nwarps) {
        const int64_t id = static_cast<int64_t>(__ldg(ids + t));
        const bool ok = vocab <= 0 || (id >= 0 && id < vocab);
        if (!ok && lane == 0 && err_flag) atomicExch(err_flag, 1);
        const uint4* src = table + (ok ? id : 0) * nv;
        for (int64_t i = lane; i < nv; i += 32)
            st_stream(out + t * nv + i, ok ? ld_stream(src + i) : make_uint4(0, 0, 0, 0));
    }
    pdl_trigger();
}

template <typename IdT>
int launch_embedding_tma(const void* table, const IdT* ids, void* out, int64_t num_tokens, int64_t hidden,
                         int64_t vocab, int32_t* err_flag, cudaStream_t st);   // embedding_tma.cu

// 1 = warp-per-row registers, 2 = TMA relay.  Both reach the same bandwidth on a large batch (the random-row
// access pattern is the limit); the relay does it with two instructions per row instead of 26 per lane, so it
// is the default for prefill-sized batches, while short batches keep the single-hop register path.
constexpr int kRelayMinTokens = 4096;

template <typename IdT>
static int launch_embedding(const void* table, const IdT* ids, void* out, int64_t num_tokens,
                            int64_t hidden, int64_t vocab, int32_t* err_flag, cudaStream_t st) {
    if (num_tokens < 0 || hidden <= 0 || (hidden % 8) != 0) return NMT_ERR_SHAPE;
    if (num_tokens == 0) return NMT_OK;
    if (!table || !ids || !out) return NMT_ERR_NULL;
    if (!aligned16(table) || !aligned16(out) || (reinterpret_cast<uintptr_t>(ids) % sizeof(IdT)) != 0 ||
        (err_flag && !aligned4(err_flag)))
        return NMT_ERR_ALIGN;
    if (tune("emb.variant", num_tokens >= kRelayMinTokens ? 2 : 1) == 2) {
        const int s = launch_embedding_tma<IdT>(table, ids, out, num_tokens, hidden, vocab, err_flag, st);
        if (s != NMT_ERR_UNSUPPORTED) return s;
    }
    const int64_t nv = hidden / 8;
    auto T = static_cast<const uint4*>(table);
    auto O = static_cast<uint4*>(out);
    int block = tune("emb.block", 256);
    block = block > 256 ? 256 : (block + 31) / 32 * 32;
    const int wpc = block / 32;
    const int per_sm = tune("emb.ctas_per_sm", 0);
    const int grid = grid_for(num_tokens, wpc, per_sm > 0 ? kSmCount * per_sm : 0x7fffffff);
    const int64_t slots = (nv + 31) / 32;
#define NMT_EMB_CASE(S) \
    launch_kernel(embedding_rowwarp_kernel<S, IdT>, grid, block, 0, st, T, ids, O, num_tokens, (int)nv, vocab, err_flag)
    if (slots <= 4) NMT_EMB_CASE(4);
    else if (slots <= 8) NMT_EMB_CASE(8);
    else if (slots <= 13) NMT_EMB_CASE(13);
    else if (slots <= 16) NMT_EMB_CASE(16);
    else launch_kernel(embedding_generic_kernel<IdT>, grid, block, 0, st, T, ids, O, num_tokens, nv, vocab, err_flag);
#undef NMT_EMB_CASE
    return finish_launch(1);
}

}  // namespace nmt

extern "C" {

int nmt_embedding_bf16_i64(const void* table, const int64_t* ids, void* out, int64_t num_tokens,
                           int64_t hidden, int64_t vocab, int32_t* err_flag, void* stream) {
    return nmt::launch_embedding<int64_t>(table, ids, out, num_tokens, hidden, vocab, err_flag,
                                          static_cast<cudaStream_t>(stream));
}
int nmt_embedding_bf16_i32(const void* table, const int32_t* ids, void* out, int64_t num_tokens,
                           int64_t hidden, int64_t vocab, int32_t* err_flag, void* stream) {
    return nmt::launch_embedding<int32_t>(table, ids, out, num_tokens, hidden, vocab, err_flag,
                                          static_cast<cudaStream_t>(stream));
}

}  // extern "C"
