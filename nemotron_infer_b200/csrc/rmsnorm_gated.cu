// Mamba-2 gated RMSNorm: g = y * silu(z); out = (g * rsqrt(mean_group(g^2) + eps)) * w.
//
// Register variant: one warp owns one (row, group) pair.  With 768 channels per
// group a group is 96 16-byte vectors = exactly 3 per lane (960 channels: 120
// vectors, 4 lane slots).  The group statistics therefore never leave the warp:
// five shuffles, no shared memory, no block barrier, no per-element division by
// the group size and no dynamically indexed accumulator array.  silu is
// evaluated once and g stays in fp32 registers between the sum of squares and
// the scaling, so y and z are read once and out is written once.
#include "nmt_common.cuh"

namespace nmt {

__device__ __forceinline__ float silu_exact(float z) { return z / (1.0f + expf(-z)); }

// TRACK: also keep the largest |output| (for the e4m3 quantiser that follows in the FP8 Mamba block,
// model/mamba_block.cuh:415-419), so that quantiser needs no maximum pass of its own.
template <int SLOTS, int RPI, bool TRACK = false>
__global__ void __launch_bounds__(256)
gated_groupwarp_kernel(const uint4* y, const uint4* z, const float* __restrict__ w, uint4* out,
                       int64_t items, int groups, int group_mask, int gv, float inv_gs, float eps,
                       unsigned int* amax_word = nullptr) {
    float amax = 0.f;
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * warps_per_cta;

    // Item i = row * groups + group starts at vector i * gv: groups tile the row.
#pragma unroll 1
    for (int64_t it0 = warp0 * RPI; it0 < items; it0 += nwarps * RPI) {
        uint4 a[RPI][SLOTS], b[RPI][SLOTS];
#pragma unroll
        for (int q = 0; q < RPI; ++q) {
            const int64_t it = it0 + q;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int v = s * 32 + lane;
                if (it < items && v < gv) {
                    a[q][s] = ld_stream(y + it * gv + v);
                    b[q][s] = ld_stream(z + it * gv + v);
                } else {
                    a[q][s] = make_uint4(0, 0, 0, 0);
                    b[q][s] = make_uint4(0, 0, 0, 0);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < RPI; ++q) {
            const int64_t it = it0 + q;
            if (it >= items) break;                       // warp-uniform
            // which group of the row this item is: a mask when the group count is a power of two (a 64-bit
            // modulo per item cost ~4 instructions per element)
            const int grp = group_mask >= 0 ? (static_cast<int>(it) & group_mask)
                                            : static_cast<int>(static_cast<uint32_t>(it % groups));
            float2 g[SLOTS][4];
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                float2 py[4], pz[4];
                unpack8x2(a[q][s], py);
                unpack8x2(b[q][s], pz);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    g[s][k] = __fmul2_rn(py[k], silu2_sfu(pz[k]));
                    acc = __ffma2_rn(g[s][k], g[s][k], acc);
                }
            }
            const float ss = warp_sum(acc.x + acc.y);
            const float rstd = rsqrtf(ss * inv_gs + eps);
            const float* wg = w + (int64_t)grp * gv * 8;
#pragma unroll
            for (int s = 0; s < SLOTS; ++s) {
                const int v = s * 32 + lane;
                if (v < gv) {
                    const uint4 o = scale8(g[s], rstd, ld_weight4(wg + v * 8), ld_weight4(wg + v * 8 + 4));
                    st_stream(out + it * gv + v, o);
                    if (TRACK) {
                        float f[8];
                        unpack8(o, f);
#pragma unroll
                        for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(f[k]));
                    }
                }
            }
        }
    }
    if (TRACK) {
        amax = warp_max(amax);
        if (lane == 0 && amax > 0.f) publish_max(amax_word, amax);
    }
    pdl_trigger();
}

// Any group size (including sizes that are not a multiple of 8, or groups too
// wide for registers): one warp per (row, group), scalar, two passes; the second
// pass re-reads the group (L1/L2-resident).  Also the fp32 twin.
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
gated_generic_kernel(const T* y, const T* z, const float* __restrict__ w, T* out,
                     int64_t items, int64_t groups, int64_t gs, float eps) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * warps_per_cta;
#pragma unroll 1
    for (int64_t it = warp0; it < items; it += nwarps) {
        const T* yg = y + it * gs;
        const T* zg = z + it * gs;
        const float* wg = w + (it % groups) * gs;
        float ss = 0.f;
        for (int64_t c = lane; c < gs; c += 32) {
            const float g = to_f32<T>(yg[c]) * silu_exact(to_f32<T>(zg[c]));
            ss = fmaf(g, g, ss);
        }
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / static_cast<float>(gs) + eps);
        for (int64_t c = lane; c < gs; c += 32) {
            const float g = to_f32<T>(yg[c]) * silu_exact(to_f32<T>(zg[c]));
            out[it * gs + c] = from_f32<T>((g * rstd) * wg[c]);
        }
    }
    pdl_trigger();
}

static int check_gated(const void* y, const void* z, const float* w, const void* out,
                       int64_t rows, int64_t cols, int64_t gs) {
    if (rows < 0 || cols <= 0 || gs <= 0 || (cols % gs) != 0) return NMT_ERR_SHAPE;
    if (rows == 0) return NMT_OK;
    if (!y || !z || !w || !out) return NMT_ERR_NULL;
    return NMT_OK;
}

// Every argument check of the bf16 form; NMT_OK means launch_gated_bf16 will launch (or rows == 0).
int validate_gated_bf16(const void* y, const void* z, const float* w, const void* out, int64_t rows, int64_t cols,
                        int64_t group_size) {
    int s = check_gated(y, z, w, out, rows, cols, group_size);
    if (s != NMT_OK || rows == 0) return s;
    if ((cols % 8) != 0) return NMT_ERR_SHAPE;
    if (!aligned16(y) || !aligned16(z) || !aligned16(out) || !aligned16(w)) return NMT_ERR_ALIGN;
    return NMT_OK;
}

int launch_gated_bf16(const void* y, const void* z, const float* w, void* out, int64_t rows, int64_t cols,
                      int64_t group_size, float eps, unsigned int* amax_word, bool* tracked, cudaStream_t st) {
    if (tracked) *tracked = false;
    int s = validate_gated_bf16(y, z, w, out, rows, cols, group_size);
    if (s != NMT_OK || rows == 0) return s;
    const int64_t groups = cols / group_size;
    const int64_t items = rows * groups;

    if ((group_size % 8) != 0 || group_size / 8 > 8 * 32) {
        const int grid = grid_for(items, 8, kSmCount * 32);
        launch_kernel(gated_generic_kernel<__nv_bfloat16>, grid, 256, 0, st, static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z), w,
            static_cast<__nv_bfloat16*>(out), items, groups, group_size, eps);
        return finish_launch(1);
    }
    const int gv = static_cast<int>(group_size / 8);
    const int slots = (gv + 31) / 32;
    int block = tune("gated.block", 128);
    block = block > 256 ? 256 : (block + 31) / 32 * 32;
    const int wpc = block / 32;
    const int rpi = tune("gated.rows_per_iter", 1);
    const int per_sm = tune("gated.ctas_per_sm", 0);
    const int grid = grid_for(items, wpc * rpi, per_sm > 0 ? kSmCount * per_sm : 0x7fffffff);
    const float inv_gs = 1.0f / static_cast<float>(group_size);
    const int gmask = (groups & (groups - 1)) == 0 ? static_cast<int>(groups - 1) : -1;
    auto Y = static_cast<const uint4*>(y);
    auto Z = static_cast<const uint4*>(z);
    auto O = static_cast<uint4*>(out);
#define NMT_GATED_CASE(S)                                                                              \
    do {                                                                                               \
        if (amax_word) { launch_kernel(gated_groupwarp_kernel<S, 1, true>, grid_for(items, wpc, per_sm > 0 ? kSmCount * per_sm : 0x7fffffff), block, 0, st, Y, Z, w, O, items, (int)groups, gmask, gv, inv_gs, eps, amax_word); if (tracked) *tracked = true; } \
        else if (rpi >= 2) launch_kernel(gated_groupwarp_kernel<S, 2>, grid, block, 0, st, Y, Z, w, O, items, (int)groups, gmask, gv, inv_gs, eps, (unsigned int*)nullptr); \
        else launch_kernel(gated_groupwarp_kernel<S, 1>, grid, block, 0, st, Y, Z, w, O, items, (int)groups, gmask, gv, inv_gs, eps, (unsigned int*)nullptr);   \
    } while (0)
    if (slots <= 1) NMT_GATED_CASE(1);
    else if (slots <= 2) NMT_GATED_CASE(2);
    else if (slots <= 3) NMT_GATED_CASE(3);
    else if (slots <= 4) NMT_GATED_CASE(4);
    else if (slots <= 6) NMT_GATED_CASE(6);
    else NMT_GATED_CASE(8);
#undef NMT_GATED_CASE
    return finish_launch(1);
}

}  // namespace nmt

extern "C" {

int nmt_rmsnorm_gated_bf16(const void* y, const void* z, const float* w, void* out,
                           int64_t rows, int64_t cols, int64_t group_size, float eps, void* stream) {
    return nmt::launch_gated_bf16(y, z, w, out, rows, cols, group_size, eps, nullptr, nullptr,
                                  static_cast<cudaStream_t>(stream));
}

int nmt_rmsnorm_gated_f32(const float* y, const float* z, const float* w, float* out,
                          int64_t rows, int64_t cols, int64_t group_size, float eps, void* stream) {
    using namespace nmt;
    int s = check_gated(y, z, w, out, rows, cols, group_size);
    if (s != NMT_OK || rows == 0) return s;
    if (!aligned4(y) || !aligned4(z) || !aligned4(out) || !aligned4(w)) return NMT_ERR_ALIGN;
    const int64_t groups = cols / group_size;
    const int64_t items = rows * groups;
    const int grid = grid_for(items, 8, kSmCount * 32);
    launch_kernel(gated_generic_kernel<float>, grid, 256, 0, static_cast<cudaStream_t>(stream), y, z, w, out, items, groups, group_size, eps);
    return finish_launch(1);
}

}  // extern "C"
