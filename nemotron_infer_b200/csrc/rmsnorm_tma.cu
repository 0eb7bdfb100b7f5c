// TMA-staged RMSNorm / residual-add + RMSNorm.
//
// A persistent CTA runs a producer/consumer ring in shared memory.  One elected
// producer thread moves tiles of C consecutive rows of x (and r) from HBM into a
// ring slot with one bulk copy per input (a tile of whole rows is one contiguous
// 16-byte-aligned range), signalling a "full" mbarrier with the byte count.  C
// consumer warps each own one row of the tile: they read it from shared memory,
// form the bf16-rounded sum, reduce the fp32 sum of squares with shuffles, scale,
// and write out_res / out straight to global memory with coalesced 16-byte
// stores; then they release the slot on an "empty" mbarrier.  Loads in flight
// are bounded by shared memory (up to ~200 KB per SM), not by registers or
// occupancy, and each activation byte still crosses HBM exactly once.
#include "nmt_tma.cuh"

namespace nmt {

NMT_DEFINE_TIMEOUT_READER();

template <int SLOTS, bool FUSE_ADD>
__global__ void __launch_bounds__(32 * 9)
norm_tma_kernel(const uint4* x, const uint4* r, const float* __restrict__ w, uint4* out_res, uint4* out,
                int64_t rows, int nv, float inv_cols, float eps, int stages) {
    pdl_wait();
    extern __shared__ __align__(128) uint8_t smem[];
    const int C = (blockDim.x >> 5) - 1;                 // consumer warps = rows per tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t row_bytes = static_cast<uint32_t>(nv) * 16u;
    const uint32_t tile_bytes = row_bytes * C;
    const uint32_t stage_bytes = tile_bytes * (FUSE_ADD ? 2u : 1u);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + stages;
    uint8_t* ring = smem + ((2 * stages * 8 + 127) / 128) * 128;   // barriers first, data 128-byte aligned
    const int64_t ntiles = (rows + C - 1) / C;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, C); }
        mbar_init_fence();
    }
    __syncthreads();

    if (warp == 0) {
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
#pragma unroll 1
            for (int64_t tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++issued) {
                const int s = issued % stages;
                const uint32_t use = issued / stages;
                if (use > 0) ok = mbar_wait(empty + s, (use - 1) & 1);
                if (!ok) break;
                const int64_t row0 = tile * C;
                const int64_t left = rows - row0;
                const uint32_t bytes = left >= C ? tile_bytes : static_cast<uint32_t>(left) * row_bytes;
                uint8_t* dst = ring + (size_t)s * stage_bytes;
                mbar_arrive_expect_tx(full + s, FUSE_ADD ? 2 * bytes : bytes);
                bulk_load(dst, x + row0 * nv, bytes, full + s);
                if (FUSE_ADD) bulk_load(dst + tile_bytes, r + row0 * nv, bytes, full + s);
            }
            // Do not leave while copies into this CTA's shared memory are still in flight: wait (bounded)
            // until the consumers have drained every slot that was filled.
            const int first = issued > stages ? issued - stages : 0;
            for (int k = first; k < issued; ++k)
                if (!mbar_wait(empty + (k % stages), (k / stages) & 1)) break;
        }
        return;
    }

    const int c = warp - 1;
    int k = 0;
#pragma unroll 1
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++k) {
        const int s = k % stages;
        if (!mbar_wait(full + s, (k / stages) & 1)) return;
        const int64_t row = tile * C + c;
        if (row < rows) {
            const uint8_t* xs = ring + (size_t)s * stage_bytes + (size_t)c * row_bytes;
            const uint8_t* rs = xs + tile_bytes;
            uint4 h[SLOTS];
            float ss = 0.f;
#pragma unroll
            for (int q = 0; q < SLOTS; ++q) {
                const int v = q * 32 + lane;
                if (v < nv) {
                    float f[8];
                    h[q] = lds128(xs + v * 16);
                    unpack8(h[q], f);
                    if (FUSE_ADD) {
                        float g[8];
                        unpack8(lds128(rs + v * 16), g);
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] += g[e];
                        h[q] = pack8(f);              // round the residual stream first
                        unpack8(h[q], f);
                        st_stream(out_res + row * nv + v, h[q]);
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
                } else {
                    h[q] = make_uint4(0, 0, 0, 0);
                }
            }
            // All shared-memory reads of this row are done: hand the slot back before the slow part.
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + s);
            ss = warp_sum(ss);
            const float rstd = rsqrtf(ss * inv_cols + eps);
#pragma unroll
            for (int q = 0; q < SLOTS; ++q) {
                const int v = q * 32 + lane;
                if (v < nv) {
                    float f[8];
                    unpack8(h[q], f);
                    const float4 w0 = ld_weight4(w + v * 8);
                    const float4 w1 = ld_weight4(w + v * 8 + 4);
                    f[0] = (f[0] * rstd) * w0.x; f[1] = (f[1] * rstd) * w0.y;
                    f[2] = (f[2] * rstd) * w0.z; f[3] = (f[3] * rstd) * w0.w;
                    f[4] = (f[4] * rstd) * w1.x; f[5] = (f[5] * rstd) * w1.y;
                    f[6] = (f[6] * rstd) * w1.z; f[7] = (f[7] * rstd) * w1.w;
                    st_stream(out + row * nv + v, pack8(f));
                }
            }
        } else {
            if (lane == 0) mbar_arrive(empty + s);
        }
    }
    pdl_trigger();
}

template <int SLOTS, bool FUSE_ADD>
static int launch_one(const uint4* X, const uint4* R, const float* w, uint4* OR, uint4* O, int64_t rows, int nv,
                      float inv_cols, float eps, int C, int stages, int grid, size_t smem, cudaStream_t st) {
    auto kern = norm_tma_kernel<SLOTS, FUSE_ADD>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynSmem) != cudaSuccess)
            return finish_launch(0);
        configured[dev] = true;
    }
    launch_kernel(kern, grid, 32 * (C + 1), smem, st, X, R, w, OR, O, rows, nv, inv_cols, eps, stages);
    return finish_launch(1);
}

// Returns NMT_ERR_UNSUPPORTED when the shape does not fit this variant (the caller then uses the register kernel).
int launch_norm_tma(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                    int64_t rows, int64_t cols, float eps, cudaStream_t st) {
    const int64_t nv64 = cols / 8;
    if (nv64 > 16 * 32) return NMT_ERR_UNSUPPORTED;
    const int nv = static_cast<int>(nv64);
    int C = tune("norm.tma_rows", 4);
    if (C < 1) C = 1;
    if (C > 8) C = 8;
    const size_t stage_bytes = (size_t)nv * 16 * C * (fuse ? 2 : 1);
    int stages = tune("norm.tma_stages", 4);
    const int per_sm = tune("norm.ctas_per_sm", 1);
    const size_t budget = (size_t)kMaxDynSmem / per_sm - (per_sm > 1 ? 1024 : 0);
    while (stages > 1 && 256 + stages * stage_bytes > budget) --stages;
    const size_t smem = ((2 * stages * 8 + 127) / 128) * 128 + stages * stage_bytes;
    if (smem > (size_t)kMaxDynSmem) return NMT_ERR_UNSUPPORTED;
    const int64_t ntiles = (rows + C - 1) / C;
    const int grid = static_cast<int>(ntiles < (int64_t)kSmCount * per_sm ? ntiles : (int64_t)kSmCount * per_sm);
    const float inv_cols = 1.0f / static_cast<float>(cols);
    auto X = static_cast<const uint4*>(x);
    auto R = static_cast<const uint4*>(r);
    auto OR = static_cast<uint4*>(out_res);
    auto O = static_cast<uint4*>(out);
    const int slots = (nv + 31) / 32;
#define NMT_TMA_CASE(S)                                                                                        \
    (fuse ? launch_one<S, true>(X, R, w, OR, O, rows, nv, inv_cols, eps, C, stages, grid, smem, st)            \
          : launch_one<S, false>(X, R, w, OR, O, rows, nv, inv_cols, eps, C, stages, grid, smem, st))
    if (slots <= 4) return NMT_TMA_CASE(4);
    if (slots <= 8) return NMT_TMA_CASE(8);
    if (slots <= 13) return NMT_TMA_CASE(13);
    return NMT_TMA_CASE(16);
#undef NMT_TMA_CASE
}

}  // namespace nmt
