// Cross-block fusion of "residual add at the tail of block i" with "pre-norm at the head of block i+1", for block
// code that stays exactly as the reference wrote it.
//
// Every reference block is  out = input + mixer(rmsnorm(input))  (model/mlp_block.cuh:98-107, model/mamba_block.cuh:
// 183-226, model/attention_block.cuh:196-213): it opens with rmsnorm_bf16 into `normed`, its FIRST workspace tensor,
// and closes with the residual add.  The add's output is re-read at once by the next block's rmsnorm, so the pair
// moves 5 tensors' worth of bytes where the fused kernel moves 4 - but the two launches sit in two different block
// calls, and neither the block signatures nor binding.cu may change.
//
// The drop-in headers therefore route the blocks' two calls through the entry points below, and the orchestrator
// (engine.py's layer loop) announces, before it calls block i, the norm weight of block i+1:
//
//   tail   nmt_block_tail_add_bf16(input, mixer, out)   with a weight announced -> ONE launch of the fused add + norm:
//          out = input + mixer, and rmsnorm(out) * next_w is written over this block's own `normed` workspace, which
//          is dead by then (its only readers, the block's first projections, precede the tail in stream order);
//   head   nmt_block_head_rmsnorm_bf16(input', normed', w')  of the next block -> NO launch when input', normed', w',
//          the shape, eps and the stream are exactly what the fused tail produced: the reference's engine rewinds its
//          bump allocator before every layer (engine.py:263, tensor/allocator.cuh:124-129), so the next block's first
//          workspace tensor is the same address and already holds its normed input.
//
// Anything that does not match (a different address after the allocator grew a slab, another stream, no
// announcement) simply runs the plain kernels: the result is the same either way, only the traffic differs.  The
// record of a fused tail is dropped by the next head call whatever its outcome, by nmt_fusion_reset(), and by ANY
// other entry point of this library that launches a kernel from this thread in between (it might have written the
// rows or the normed tensor): a head is skipped only when it is the very next launch after the fused tail.
// State is per host thread (the reference drives its layers from one thread, binding.cu holds the GIL).
#include "nmt_common.cuh"

namespace nmt {

struct NormRecord {
    const void* x = nullptr;      // the rows that were (or are to be) normed
    void* y = nullptr;            // where their normed form lives
    const float* w = nullptr;
    int64_t rows = 0, cols = 0;
    float eps = 0.f;
    cudaStream_t st = nullptr;
    int64_t epoch = 0;            // thread_launch_epoch() right after the launch that produced y
    bool valid = false;
};
struct FusionState {
    const float* next_w = nullptr;   // announced by nmt_fuse_next_norm, consumed by the next tail add
    float next_eps = 0.f;
    bool armed = false;
    NormRecord head;                 // this block's head norm: y is the block's `normed` workspace
    NormRecord ready;                // a fused tail's product: rows of x are already normed into y with w
    int64_t fused_tails = 0, elided_heads = 0;
};
static thread_local FusionState t_fusion;

}  // namespace nmt

extern "C" {

int nmt_fuse_next_norm(const float* next_norm_w, float eps) {
    nmt::FusionState& f = nmt::t_fusion;
    if (next_norm_w && !nmt::aligned16(next_norm_w)) return NMT_ERR_ALIGN;
    f.next_w = next_norm_w;
    f.next_eps = eps;
    f.armed = next_norm_w != nullptr;
    return NMT_OK;
}

int nmt_fusion_reset(void) {
    nmt::FusionState& f = nmt::t_fusion;
    f.armed = false;
    f.head.valid = false;
    f.ready.valid = false;
    return NMT_OK;
}

int nmt_fusion_counters(int64_t* fused_tails, int64_t* elided_heads) {
    if (fused_tails) *fused_tails = nmt::t_fusion.fused_tails;
    if (elided_heads) *elided_heads = nmt::t_fusion.elided_heads;
    return NMT_OK;
}

int nmt_block_head_rmsnorm_bf16(const void* x, void* y, const float* w, int64_t rows, int64_t cols, float eps,
                                void* stream) {
    nmt::FusionState& f = nmt::t_fusion;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const nmt::NormRecord r = f.ready;
    f.ready.valid = false;                       // one use only, whatever happens next
    f.head.valid = false;
    const bool done_already = r.valid && rows > 0 && r.x == x && r.y == y && r.w == w && r.rows == rows &&
                              r.cols == cols && r.eps == eps && r.st == st && r.epoch == nmt::thread_launch_epoch();
    if (!done_already) {
        const int s = nmt_rmsnorm_bf16(x, y, w, rows, cols, eps, stream);
        if (s != NMT_OK) return s;
    } else {
        ++f.elided_heads;                        // the previous block's tail wrote exactly this tensor
    }
    if (rows > 0) {
        f.head.x = x; f.head.y = y; f.head.w = w; f.head.rows = rows; f.head.cols = cols; f.head.eps = eps; f.head.st = st;
        f.head.valid = true;
    }
    return NMT_OK;
}

int nmt_block_tail_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream) {
    nmt::FusionState& f = nmt::t_fusion;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool armed = f.armed;
    const nmt::NormRecord h = f.head;
    f.armed = false;                             // an announcement serves one tail
    f.head.valid = false;
    f.ready.valid = false;
    if (armed && h.valid && n > 0 && n == h.rows * h.cols && st == h.st && out != h.y && a != h.y && b != h.y) {
        const int s = nmt_add_rmsnorm_bf16(a, b, f.next_w, out, h.y, h.rows, h.cols, f.next_eps, stream);
        if (s == NMT_OK) {
            f.ready.x = out; f.ready.y = h.y; f.ready.w = f.next_w; f.ready.rows = h.rows; f.ready.cols = h.cols;
            f.ready.eps = f.next_eps; f.ready.st = st; f.ready.epoch = nmt::thread_launch_epoch(); f.ready.valid = true;
            ++f.fused_tails;
            return NMT_OK;
        }
        // the fused form refused these arguments (nothing was launched): fall back to the plain add
    }
    return nmt_add_bf16(a, b, out, n, stream);
}

}  // extern "C"
