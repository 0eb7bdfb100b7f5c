// RMSNorm and fused residual-add + RMSNorm.
//
// Default kernel (rows up to 32,768 columns): one CTA per row, the row spread over ~96-160 threads that each hold
// 3-5 16-byte vectors of x (and r) in registers.  All loads of a row are issued before the first use, the rounded
// sum x + r stays in registers between the sum of squares and the scaling, the row statistic costs five shuffles
// plus one block barrier, and every activation byte crosses HBM once: read x, read r, write out_res, write out.
// Wider rows go to the cluster kernels in rmsnorm_cluster.cu; the two-pass kernel below is the last resort.
#include "nmt_common.cuh"

namespace nmt {

// CTA-per-row register variant: blockDim threads share ROWS consecutive rows (thread t owns vectors t,
// t + blockDim, ... of each), so each thread holds only SLOTS = ceil(vectors / blockDim) vectors of x and r per
// row.  Few registers per thread means many resident warps (the occupancy the memory system needs), and the
// price is one block barrier per row group for the sum of squares.  Partial sums are added in a fixed order,
// so results are deterministic.  The arithmetic runs on register pairs (add.bf16x2 for the residual sum, which
// rounds the exact sum once exactly like "add in fp32, round to bf16"; f32x2 fma / mul for the rest).
template <int SLOTS, int ROWS, bool FUSE_ADD>
__global__ void __launch_bounds__(512)
rmsnorm_ctarow_kernel(const uint4* x, const uint4* r, const float* __restrict__ w, uint4* out_res, uint4* out,
                      int64_t rows, int nv, float inv_cols, float eps) {
    pdl_wait();
    __shared__ __align__(16) float s_part[2][ROWS][16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int flip = 0;
#pragma unroll 1
    for (int64_t row0 = (int64_t)blockIdx.x * ROWS; row0 < rows; row0 += (int64_t)gridDim.x * ROWS, flip ^= 1) {
        uint4 a[ROWS][SLOTS], b[ROWS][SLOTS];
#pragma unroll
        for (int q = 0; q < ROWS; ++q) {
            const int64_t row = row0 + q;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int v = s * blockDim.x + threadIdx.x;
                if (row < rows && v < nv) {
                    a[q][s] = ld_stream(x + row * nv + v);
                    if (FUSE_ADD) b[q][s] = ld_stream(r + row * nv + v);
                } else {
                    a[q][s] = make_uint4(0, 0, 0, 0);
                    if (FUSE_ADD) b[q][s] = make_uint4(0, 0, 0, 0);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < ROWS; ++q) {
            const int64_t row = row0 + q;
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                if (FUSE_ADD) {
                    // The residual stream is rounded to bf16 first: the norm must see what the next block
                    // would read back from memory.
                    a[q][s] = add_bf16x8_rn(a[q][s], b[q][s]);
                    const int v = s * blockDim.x + threadIdx.x;
                    if (row < rows && v < nv) st_stream(out_res + row * nv + v, a[q][s]);
                }
                float2 p[4];
                unpack8x2(a[q][s], p);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc = __ffma2_rn(p[k], p[k], acc);
            }
            const float ss = warp_sum(acc.x + acc.y);
            if (lane == 0) s_part[flip][q][wid] = ss;
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < ROWS; ++q) {
            const int64_t row = row0 + q;
            if (row >= rows) break;
            float total = 0.f;
            for (int i = 0; i < nwarps; ++i) total += s_part[flip][q][i];
            const float rstd = rsqrtf(total * inv_cols + eps);
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int v = s * blockDim.x + threadIdx.x;
                if (v < nv) {
                    float2 p[4];
                    unpack8x2(a[q][s], p);
                    st_stream(out + row * nv + v, scale8(p, rstd, ld_weight4(w + v * 8), ld_weight4(w + v * 8 + 4)));
                }
            }
        }
    }
    pdl_trigger();
}

// Any width: one CTA per row, two passes.  The second pass re-reads what the
// first pass of the same thread touched (out_res when fused, else x), so the
// re-read is served by L2 for all but pathological widths.
template <bool FUSE_ADD>
__global__ void __launch_bounds__(256)
rmsnorm_rowcta_kernel(const uint4* x, const uint4* r,
                      const float* __restrict__ w, uint4* out_res, uint4* out,
                      int64_t rows, int64_t nv, float inv_cols, float eps) {
    pdl_wait();
    __shared__ float s_part[8];
    __shared__ float s_total;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll 1
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint4* xr = x + row * nv;
        float ss = 0.f;
        for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
            uint4 a = ld_stream(xr + v);
            float f[8];
            unpack8(a, f);
            if (FUSE_ADD) {
                float g[8];
                unpack8(ld_stream(r + row * nv + v), g);
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] += g[k];
                a = pack8(f);
                unpack8(a, f);
                out_res[row * nv + v] = a;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss = fmaf(f[k], f[k], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[wid] = ss;
        __syncthreads();
        if (wid == 0) {
            float t = lane < (blockDim.x >> 5) ? s_part[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) s_total = t;
        }
        __syncthreads();
        const float rstd = rsqrtf(s_total * inv_cols + eps);
        const uint4* src = FUSE_ADD ? out_res + row * nv : xr;
        for (int64_t v = threadIdx.x; v < nv; v += blockDim.x) {
            float f[8];
            unpack8(src[v], f);
            const float4 w0 = ld_weight4(w + v * 8);
            const float4 w1 = ld_weight4(w + v * 8 + 4);
            f[0] = (f[0] * rstd) * w0.x; f[1] = (f[1] * rstd) * w0.y;
            f[2] = (f[2] * rstd) * w0.z; f[3] = (f[3] * rstd) * w0.w;
            f[4] = (f[4] * rstd) * w1.x; f[5] = (f[5] * rstd) * w1.y;
            f[6] = (f[6] * rstd) * w1.z; f[7] = (f[7] * rstd) * w1.w;
            out[row * nv + v] = pack8(f);
        }
        __syncthreads();   // s_part / s_total are reused by the next row
    }
    pdl_trigger();
}

// fp32 twin (parity only): one CTA per row, scalar, two passes.
__global__ void __launch_bounds__(256)
rmsnorm_f32_kernel(const float* __restrict__ x, float* y, const float* __restrict__ w,
                   int64_t rows, int64_t cols, float eps) {
    pdl_wait();
    __shared__ float s_part[8];
    __shared__ float s_total;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll 1
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float* xr = x + row * cols;
        float ss = 0.f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) { const float v = xr[c]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) s_part[wid] = ss;
        __syncthreads();
        if (wid == 0) {
            float t = lane < (blockDim.x >> 5) ? s_part[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) s_total = t;
        }
        __syncthreads();
        const float rstd = rsqrtf(s_total / static_cast<float>(cols) + eps);
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) y[row * cols + c] = (xr[c] * rstd) * w[c];
        __syncthreads();
    }
    pdl_trigger();
}

int launch_norm_cluster(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                        int64_t rows, int64_t cols, float eps, int cluster, cudaStream_t st);   // rmsnorm_cluster.cu
int launch_norm_staged_single(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                              int64_t rows, int64_t cols, float eps, cudaStream_t st);           // rmsnorm_cluster.cu

template <bool FUSE_ADD>
static int launch_norm_bf16(const void* x, const void* r, const float* w, void* out_res, void* out,
                            int64_t rows, int64_t cols, float eps, cudaStream_t st) {
    const int64_t nv = cols / 8;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    auto X = static_cast<const uint4*>(x);
    auto R = static_cast<const uint4*>(r);
    auto OR = static_cast<uint4*>(out_res);
    auto O = static_cast<uint4*>(out);

    // norm.cluster: 0 = a cluster of CTAs per row where one CTA cannot hold the row in registers (more than 32,768
    // columns), 2 / 4 / 8 = that cluster size for every width, 1 = never (wide rows take the two-pass kernel).
    const int cluster = tune("norm.cluster", 0);
    if (cluster >= 2 || (cluster == 0 && nv > 8 * 512)) {
        const int s = launch_norm_cluster(FUSE_ADD, x, r, w, out_res, out, rows, cols, eps, cluster, st);
        if (s != NMT_ERR_UNSUPPORTED) return s;
    }
    if (!FUSE_ADD && cluster == 0 && nv > 2560 && nv <= 8 * 512 && tune("norm.staged_single", 1) == 1) {
        const int s = launch_norm_staged_single(false, x, r, w, out_res, out, rows, cols, eps, st);
        if (s != NMT_ERR_UNSUPPORTED) return s;
    }
    if (nv <= 8 * 512) {
        // Default shape: about 160 threads per row (392 vectors -> 3 per thread), at most 8 vectors per thread.
        int block = tune("norm.block", 0);
        if (block <= 0) block = default_norm_block(nv, FUSE_ADD);
        block = block > 512 ? 512 : (block + 31) / 32 * 32;
        if ((nv + block - 1) / block > 8) block = 512;     // a swept block size too small for this width
        const int slots = static_cast<int>((nv + block - 1) / block);
        const int per_sm = tune("norm.ctas_per_sm", 0);
        const int rows_per_cta = tune("norm.rows_per_cta", 1);
        const int rows_used = (rows_per_cta >= 4 && !FUSE_ADD && slots <= 4) ? 4 : rows_per_cta >= 2 ? 2 : 1;
        const int grid = grid_for(rows, rows_used, per_sm > 0 ? kSmCount * per_sm : 0x7fffffff);
#define NMT_CTAROW_CASE(S)                                                                                   \
    do {                                                                                                     \
        if (rows_per_cta >= 4 && !FUSE_ADD && S <= 4) launch_kernel(rmsnorm_ctarow_kernel<S, 4, false>, grid, block, 0, st, X, R, w, OR, O, rows, (int)nv, inv_cols, eps); \
        else if (rows_per_cta >= 2) launch_kernel(rmsnorm_ctarow_kernel<S, 2, FUSE_ADD>, grid, block, 0, st, X, R, w, OR, O, rows, (int)nv, inv_cols, eps); \
        else launch_kernel(rmsnorm_ctarow_kernel<S, 1, FUSE_ADD>, grid, block, 0, st, X, R, w, OR, O, rows, (int)nv, inv_cols, eps);                   \
    } while (0)
        if (slots <= 1) NMT_CTAROW_CASE(1);
        else if (slots <= 2) NMT_CTAROW_CASE(2);
        else if (slots <= 3) NMT_CTAROW_CASE(3);
        else if (slots <= 4) NMT_CTAROW_CASE(4);
        else if (slots <= 5) NMT_CTAROW_CASE(5);
        else if (slots <= 7) NMT_CTAROW_CASE(7);
        else NMT_CTAROW_CASE(8);
#undef NMT_CTAROW_CASE
        return finish_launch(1);
    }
    // Wider than one CTA's registers and no cluster launch possible: one CTA per row, two passes.
    const int grid = grid_for(rows, 1, kSmCount * 16);
    launch_kernel(rmsnorm_rowcta_kernel<FUSE_ADD>, grid, 256, 0, st, X, R, w, OR, O, rows, nv, inv_cols, eps);
    return finish_launch(1);
}

static int check_norm_args(const void* x, const void* y, const float* w, int64_t rows, int64_t cols) {
    if (rows < 0 || cols <= 0 || (cols % 8) != 0) return NMT_ERR_SHAPE;
    if (rows == 0) return NMT_OK;
    if (!x || !y || !w) return NMT_ERR_NULL;
    if (!aligned16(x) || !aligned16(y) || !aligned16(w)) return NMT_ERR_ALIGN;
    return NMT_OK;
}

}  // namespace nmt

extern "C" {

int nmt_rmsnorm_f32(const float* x, float* y, const float* w, int64_t rows, int64_t cols, float eps, void* stream) {
    if (rows < 0 || cols <= 0) return NMT_ERR_SHAPE;
    if (rows == 0) return NMT_OK;
    if (!x || !y || !w) return NMT_ERR_NULL;
    if (!nmt::aligned4(x) || !nmt::aligned4(y) || !nmt::aligned4(w)) return NMT_ERR_ALIGN;
    const int grid = nmt::grid_for(rows, 1, nmt::kSmCount * 8);
    nmt::launch_kernel(nmt::rmsnorm_f32_kernel, grid, 256, 0, static_cast<cudaStream_t>(stream), x, y, w, rows, cols, eps);
    return nmt::finish_launch(1);
}

int nmt_rmsnorm_bf16(const void* x, void* y, const float* w, int64_t rows, int64_t cols, float eps, void* stream) {
    int s = nmt::check_norm_args(x, y, w, rows, cols);
    if (s != NMT_OK || rows == 0) return s;
    return nmt::launch_norm_bf16<false>(x, nullptr, w, nullptr, y, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

int nmt_add_rmsnorm_bf16(const void* x, const void* r, const float* w, void* out_res, void* out,
                         int64_t rows, int64_t cols, float eps, void* stream) {
    int s = nmt::check_norm_args(x, out, w, rows, cols);
    if (s != NMT_OK || rows == 0) return s;
    if (!r || !out_res) return NMT_ERR_NULL;
    if (!nmt::aligned16(r) || !nmt::aligned16(out_res)) return NMT_ERR_ALIGN;
    if (out == x || out == r || out == out_res) return NMT_ERR_SHAPE;
    return nmt::launch_norm_bf16<true>(x, r, w, out_res, out, rows, cols, eps, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
