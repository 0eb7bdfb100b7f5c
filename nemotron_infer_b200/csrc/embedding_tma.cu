// Token-embedding gather as a TMA relay: rows never pass through registers.
//
// Each warp is a relay with its own ring of STAGES row slots in shared memory.  Its elected lane issues one
// bulk copy table[id] -> slot (6272 bytes for the 3136-wide table, completion on the slot's mbarrier) and,
// LAG rows later, one bulk copy slot -> out[token].  A slot is refilled only after the bulk store that read
// it has finished reading (cp.async.bulk.wait_group.read).  The copy engine does the address generation,
// so the SM issues two instructions per row instead of 26 loads/stores per lane, and the bytes in flight
// (LAG rows per relay) are bounded by shared memory rather than by registers.
//
// Ids outside [0, vocab) are never dereferenced: the relay zero-fills the slot itself and raises *err_flag.
#include "nmt_tma.cuh"

namespace nmt {

NMT_DEFINE_TIMEOUT_READER();

constexpr int kIdBlock = 8;     // tokens per id fetch (lanes 0..7 load one id each)

template <int STAGES, typename IdT>
__global__ void __launch_bounds__(256)
embedding_relay_kernel(const uint8_t* __restrict__ table, const IdT* __restrict__ ids, uint8_t* __restrict__ out,
                       int64_t num_tokens, uint32_t row_bytes, uint32_t slot_stride, int64_t vocab, int32_t* err_flag) {
    pdl_wait();
    constexpr int LAG = STAGES / 2;
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem) + warp * STAGES;
    uint8_t* ring = smem + ((nwarps * STAGES * 8 + 127) / 128) * 128 + (size_t)warp * STAGES * slot_stride;

    if (lane == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(full + s, 1);
        mbar_init_fence();
    }
    __syncwarp();

    const int64_t relay = (int64_t)blockIdx.x * nwarps + warp;
    const int64_t nrelays = (int64_t)gridDim.x * nwarps;
    const int64_t nblocks = (num_tokens + kIdBlock - 1) / kIdBlock;
    const int64_t my_blocks = nblocks > relay ? (nblocks - relay + nrelays - 1) / nrelays : 0;
    const int64_t my_chunks = my_blocks * kIdBlock;
    bool alive = true;
    int64_t my_id = 0;
    int64_t filled = 0, stored = 0;     // chunks whose slot fill was started / whose row was handed to a bulk store

    for (int64_t i = 0; i < my_chunks + LAG && alive; ++i) {
        if (i < my_chunks) {
            const int64_t blk = relay + (i / kIdBlock) * nrelays;
            const int k = static_cast<int>(i % kIdBlock);
            if (k == 0) {
                const int64_t t = blk * kIdBlock + lane;
                my_id = (lane < kIdBlock && t < num_tokens) ? static_cast<int64_t>(__ldg(ids + t)) : 0;
            }
            const int64_t id = __shfl_sync(0xffffffffu, my_id, k);
            const int64_t tok = blk * kIdBlock + k;
            if (tok < num_tokens) {
                const int s = static_cast<int>(i % STAGES);
                uint8_t* slot = ring + (size_t)s * slot_stride;
                if (i >= STAGES && lane == 0) bulk_wait_read<STAGES - LAG - 1>();   // store of chunk i-STAGES has read the slot
                __syncwarp();
                const bool ok = vocab <= 0 || (id >= 0 && id < vocab);
                if (ok) {
                    if (lane == 0) {
                        mbar_arrive_expect_tx(full + s, row_bytes);
                        bulk_load(slot, table + (size_t)id * row_bytes, row_bytes, full + s);
                    }
                } else {
                    for (uint32_t b = lane * 16; b < row_bytes; b += 32 * 16) sts128(slot + b, make_uint4(0, 0, 0, 0));
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (err_flag) atomicExch(err_flag, 1);
                        mbar_arrive(full + s);
                    }
                }
                filled = i + 1;
            }
        }
        const int64_t j = i - LAG;
        if (j >= 0) {
            const int64_t tok = (relay + (j / kIdBlock) * nrelays) * kIdBlock + (j % kIdBlock);
            if (tok < num_tokens) {
                const int s = static_cast<int>(j % STAGES);
                if (lane == 0) {
                    alive = mbar_wait(full + s, static_cast<uint32_t>(j / STAGES) & 1u);
                    if (alive) {
                        bulk_store(out + (size_t)tok * row_bytes, ring + (size_t)s * slot_stride, row_bytes);
                        bulk_commit();
                        stored = j + 1;
                    }
                }
                alive = __shfl_sync(0xffffffffu, alive, 0);
            }
        }
    }
    // A wait ran out (counted; the results are void): bulk loads into this relay's slots may still be in flight.
    // Wait, bounded again, for every slot that was filled and never stored, so that no copy lands in shared
    // memory after the CTA has left.
    if (!alive && lane == 0) {
        for (int64_t c = stored; c < filled; ++c)
            mbar_wait(full + static_cast<int>(c % STAGES), static_cast<uint32_t>(c / STAGES) & 1u);
    }
    // Shared memory must outlive every bulk store that reads it.
    if (lane == 0) bulk_wait_all<0>();
    pdl_trigger();
}

template <int STAGES, typename IdT>
static int launch_relay(const void* table, const IdT* ids, void* out, int64_t num_tokens, int64_t hidden,
                        int64_t vocab, int32_t* err_flag, cudaStream_t st) {
    const uint32_t row_bytes = static_cast<uint32_t>(hidden * 2);
    const uint32_t slot_stride = (row_bytes + 127u) / 128u * 128u;
    int warps = tune("emb.relay_warps", 4);
    if (warps < 1) warps = 1;
    if (warps > 8) warps = 8;
    while (warps > 1 && (size_t)warps * STAGES * slot_stride + 1024 > (size_t)kMaxDynSmem) --warps;
    const size_t smem = ((warps * STAGES * 8 + 127) / 128) * 128 + (size_t)warps * STAGES * slot_stride;
    if (smem > (size_t)kMaxDynSmem) return NMT_ERR_UNSUPPORTED;
    // More CTAs than fit at once: the block scheduler then evens out the tail (measured best at 8 per SM).
    const int per_sm = tune("emb.ctas_per_sm", 8);
    const int64_t nblocks = (num_tokens + kIdBlock - 1) / kIdBlock;
    int64_t grid = (nblocks + warps - 1) / warps;
    if (grid > (int64_t)kSmCount * per_sm) grid = (int64_t)kSmCount * per_sm;
    auto kern = embedding_relay_kernel<STAGES, IdT>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess)
            return finish_launch(0);
        configured[dev] = true;
    }
    launch_kernel(kern, static_cast<int>(grid), warps * 32, smem, st, static_cast<const uint8_t*>(table), ids,
                                                         static_cast<uint8_t*>(out), num_tokens, row_bytes,
                                                         slot_stride, vocab, err_flag);
    return finish_launch(1);
}

template <typename IdT>
int launch_embedding_tma(const void* table, const IdT* ids, void* out, int64_t num_tokens, int64_t hidden,
                         int64_t vocab, int32_t* err_flag, cudaStream_t st) {
    if (hidden * 2 > 64 * 1024) return NMT_ERR_UNSUPPORTED;      // one slot must fit comfortably
    const int stages = tune("emb.tma_stages", 4);
    if (stages >= 8) return launch_relay<8, IdT>(table, ids, out, num_tokens, hidden, vocab, err_flag, st);
    if (stages >= 4) return launch_relay<4, IdT>(table, ids, out, num_tokens, hidden, vocab, err_flag, st);
    return launch_relay<2, IdT>(table, ids, out, num_tokens, hidden, vocab, err_flag, st);
}

template int launch_embedding_tma<int32_t>(const void*, const int32_t*, void*, int64_t, int64_t, int64_t, int32_t*, cudaStream_t);
template int launch_embedding_tma<int64_t>(const void*, const int64_t*, void*, int64_t, int64_t, int64_t, int32_t*, cudaStream_t);

}  // namespace nmt
