// W8A16 GEMV for single-token decode: y[n] = (sum_k e4m3(W[n,k]) * bf16(x[k])) * w_scale[n].
//
// With one token the projection is pure weight streaming (24-55 MB of e4m3 per matrix, 5.4 GB per token for the
// whole model, ops/gemv.cuh:4-6): the only thing that matters is how fast W crosses HBM, and a matrix is gone in
// a few microseconds, so every SM has to have deep loads in flight from its first cycle.
//   * Persistent grid, one CTA of 8 warps per SM slot.  x is converted to fp32 once per CTA into shared memory
//     (16 floats per 16 weights come back as four LDS.128, no per-use unpacking).
//   * A work unit is (row, K-slice): rows are cut into SPLIT slices of ~3 KB so that short-and-wide matrices
//     (down_proj: 3136 rows of 12544) still give every warp several units; the SPLIT warps that share a row sit
//     in one CTA and combine their partial sums through shared memory in a fixed order (deterministic).
//   * Each lane issues all 16-byte weight loads of its unit before the first use, and the next unit's before the
//     arithmetic of the current one; consecutive lanes read consecutive 16 bytes.  e4m3 pairs go to f16x2 with
//     one cvt (exact), then to fp32, and accumulate with f32x2 FMAs in fp32 -- the arithmetic the reference
//     specifies (ops/gemv.cuh:20-22), no fp16 accumulation.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "nmt_common.cuh"

namespace nmt {

constexpr int kGemvWarps = 8;

// 4 e4m3 bytes (one 32-bit word) -> 4 floats, as two (lo, hi) pairs.
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t wd, float2& a, float2& b) {
    uint32_t h0, h1;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h0) : "h"(static_cast<unsigned short>(wd & 0xffffu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h1) : "h"(static_cast<unsigned short>(wd >> 16)));
    a = __half22float2(*reinterpret_cast<__half2*>(&h0));
    b = __half22float2(*reinterpret_cast<__half2*>(&h1));
}

// 16 weights (vector v of the row) against their 16 activations.  x sits in shared memory as fp32 in four
// planes: plane j holds elements 4j..4j+3 of every 16-element vector, so that the 32 lanes of a warp (consecutive
// v) read consecutive float4s -- the straightforward [v][16] layout made every LDS.128 a four-way bank conflict
// (73 % of all shared-memory wavefronts in the first version were conflict replays).
__device__ __forceinline__ float2 dot16(const uint4& wv, const float4* xs, int v, int kv, float2 acc) {
    const float4 x0 = xs[v];
    const float4 x1 = xs[kv + v];
    const float4 x2 = xs[2 * kv + v];
    const float4 x3 = xs[3 * kv + v];
    float2 a, b;
    e4m3x4_to_f32(wv.x, a, b);
    acc = __ffma2_rn(a, make_float2(x0.x, x0.y), acc);
    acc = __ffma2_rn(b, make_float2(x0.z, x0.w), acc);
    e4m3x4_to_f32(wv.y, a, b);
    acc = __ffma2_rn(a, make_float2(x1.x, x1.y), acc);
    acc = __ffma2_rn(b, make_float2(x1.z, x1.w), acc);
    e4m3x4_to_f32(wv.z, a, b);
    acc = __ffma2_rn(a, make_float2(x2.x, x2.y), acc);
    acc = __ffma2_rn(b, make_float2(x2.z, x2.w), acc);
    e4m3x4_to_f32(wv.w, a, b);
    acc = __ffma2_rn(a, make_float2(x3.x, x3.y), acc);
    acc = __ffma2_rn(b, make_float2(x3.z, x3.w), acc);
    return acc;
}

constexpr int kGemvMaxIters = 32;  // passes a CTA of the unit kernel may make when rows are split (sizes its smem)
constexpr int kGemvSlots = 8;     // 16-byte vectors per lane per work unit: a unit is at most 8 * 32 * 16 = 4096 weights

// Unit kernel: a work unit (row, K-slice) of at most 4096 weights is loaded WHOLE, every lane issuing all of its
// 16-byte loads at once, and the next unit's loads are issued before the current unit's arithmetic, so a warp
// pays one memory latency in total instead of one per handful of loads.  The first unit is requested before x
// is staged, which hides the staging behind the first trip to HBM.
template <int SPLIT>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_w8a16_unit_kernel(const __nv_bfloat16* __restrict__ x, const uint4* __restrict__ W, const float* __restrict__ w_scale,
                       __nv_bfloat16* __restrict__ y, int N, int kv /* 16-byte vectors per row */) {
    pdl_wait();
    extern __shared__ __align__(16) float smem_f[];
    float* xs_w = smem_f;                                  // K floats, in four planes (see dot16)
    const float4* xs = reinterpret_cast<const float4*>(smem_f);
    float* part = smem_f + (size_t)kv * 16;                // kGemvWarps partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int ROWS_PER_CTA = kGemvWarps / SPLIT;
    const int slice = warp % SPLIT, row_in_cta = warp / SPLIT;
    const int v_per_slice = (kv + SPLIT - 1) / SPLIT;
    const int v0 = slice * v_per_slice;
    const int v1 = min(v0 + v_per_slice, kv);
    const int stride = gridDim.x * ROWS_PER_CTA;

    auto fetch = [&](int row, uint4 (&w)[kGemvSlots]) {
        const uint4* wr = W + (size_t)row * kv;
#pragma unroll
        for (int s = 0; s < kGemvSlots; ++s) {
            const int v = v0 + s * 32 + lane;
            w[s] = (row < N && v < v1) ? ld_stream(wr + v) : make_uint4(0, 0, 0, 0);
        }
    };
    int row = blockIdx.x * ROWS_PER_CTA + row_in_cta;
    uint4 cur[kGemvSlots], nxt[kGemvSlots];
    fetch(row, cur);
    for (int i = threadIdx.x; i < kv * 8; i += blockDim.x) {            // two bf16 per step
        const uint32_t u = reinterpret_cast<const uint32_t*>(x)[i];
        const int k = 2 * i, vec = k >> 4, j = (k >> 2) & 3, e = k & 3;    // element k -> plane j, vector vec, slot e
        xs_w[((size_t)j * kv + vec) * 4 + e] = bf16_lo(u);
        xs_w[((size_t)j * kv + vec) * 4 + e + 1] = bf16_hi(u);
    }
    __syncthreads();
    // With K-slices the SPLIT warps of a row meet in shared memory.  Their partial sums are parked per iteration
    // (the launcher sizes the grid so that a CTA makes at most kGemvMaxIters passes) and combined after ONE block
    // barrier at the end, instead of two barriers per row.
    int it = 0;
#pragma unroll 1
    for (int row0 = blockIdx.x * ROWS_PER_CTA; row0 < N; row0 += stride, row += stride, ++it) {
        fetch(row + stride, nxt);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int s = 0; s < kGemvSlots; ++s) {
            const int v = v0 + s * 32 + lane;
            if (v < v1) acc = dot16(cur[s], xs, v, kv, acc);
        }
        const float sum = warp_sum(acc.x + acc.y);
        if (SPLIT > 1) {
            if (lane == 0) part[it * kGemvWarps + warp] = sum;
        } else if (lane == 0 && row < N) {
            y[row] = __float2bfloat16_rn(sum * __ldg(w_scale + row));
        }
#pragma unroll
        for (int s = 0; s < kGemvSlots; ++s) cur[s] = nxt[s];
    }
    if (SPLIT > 1) {
        __syncthreads();
        // rows_in_flight = it * ROWS_PER_CTA results; thread t finishes result t (fixed summation order)
        for (int r = threadIdx.x; r < it * ROWS_PER_CTA; r += blockDim.x) {
            const int i = r / ROWS_PER_CTA, rc = r % ROWS_PER_CTA;
            const int orow = (blockIdx.x + i * gridDim.x) * ROWS_PER_CTA + rc;
            if (orow < N) {
                float t = 0.f;
#pragma unroll
                for (int k = 0; k < SPLIT; ++k) t += part[i * kGemvWarps + rc * SPLIT + k];
                y[orow] = __float2bfloat16_rn(t * __ldg(w_scale + orow));
            }
        }
    }
    pdl_trigger();
}

// Loop kernel: any slice length (rows longer than 8 * 4096 weights); UNROLL loads in flight per lane.
template <int SPLIT, int UNROLL>
__global__ void __launch_bounds__(kGemvWarps * 32)
gemv_w8a16_kernel(const __nv_bfloat16* __restrict__ x, const uint4* __restrict__ W, const float* __restrict__ w_scale,
                  __nv_bfloat16* __restrict__ y, int N, int kv /* 16-byte vectors per row */) {
    pdl_wait();
    extern __shared__ __align__(16) float smem_f[];
    float* xs_w = smem_f;                                  // K floats, in four planes (see dot16)
    const float4* xs = reinterpret_cast<const float4*>(smem_f);
    float* part = smem_f + (size_t)kv * 16;                // kGemvWarps partial sums
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < kv * 8; i += blockDim.x) {            // two bf16 per step
        const uint32_t u = reinterpret_cast<const uint32_t*>(x)[i];
        const int k = 2 * i, vec = k >> 4, j = (k >> 2) & 3, e = k & 3;    // element k -> plane j, vector vec, slot e
        xs_w[((size_t)j * kv + vec) * 4 + e] = bf16_lo(u);
        xs_w[((size_t)j * kv + vec) * 4 + e + 1] = bf16_hi(u);
    }
    __syncthreads();

    constexpr int ROWS_PER_CTA = kGemvWarps / SPLIT;       // rows a CTA works on at once
    const int slice = warp % SPLIT;                        // which K-slice of the row this warp owns
    const int row_in_cta = warp / SPLIT;
    const int v_per_slice = (kv + SPLIT - 1) / SPLIT;
    const int v0 = slice * v_per_slice;
    const int v1 = min(v0 + v_per_slice, kv);
#pragma unroll 1
    for (int row0 = blockIdx.x * ROWS_PER_CTA; row0 < N; row0 += gridDim.x * ROWS_PER_CTA) {
        const int row = row0 + row_in_cta;
        float2 acc = make_float2(0.f, 0.f);
        if (row < N) {
            const uint4* wr = W + (size_t)row * kv;
            int v = v0 + lane;
            for (; v + 32 * (UNROLL - 1) < v1; v += 32 * UNROLL) {
                uint4 w[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) w[u] = ld_stream(wr + v + 32 * u);
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) acc = dot16(w[u], xs, v + 32 * u, kv, acc);
            }
            for (; v < v1; v += 32) acc = dot16(ld_stream(wr + v), xs, v, kv, acc);
        }
        float s = warp_sum(acc.x + acc.y);
        if (SPLIT > 1) {
            if (lane == 0) part[warp] = s;
            __syncthreads();
            if (slice == 0 && lane == 0 && row < N) {
                float t = 0.f;
#pragma unroll
                for (int k = 0; k < SPLIT; ++k) t += part[warp + k];
                y[row] = __float2bfloat16_rn(t * __ldg(w_scale + row));
            }
            __syncthreads();
        } else if (lane == 0 && row < N) {
            y[row] = __float2bfloat16_rn(s * __ldg(w_scale + row));
        }
    }
    pdl_trigger();
}

template <int SPLIT>
static int launch_gemv(const void* x, const void* W, const float* w_scale, void* y, int N, int kv, cudaStream_t st) {
    constexpr int UNROLL = 4;
    const bool unit = (kv + SPLIT - 1) / SPLIT <= kGemvSlots * 32 && tune("gemv.variant", 1) == 1;
    auto kern = unit ? gemv_w8a16_unit_kernel<SPLIT> : gemv_w8a16_kernel<SPLIT, UNROLL>;
    const size_t smem = (size_t)kv * 16 * sizeof(float) + kGemvWarps * kGemvMaxIters * sizeof(float);
    static bool configured[2][64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !configured[unit][dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return finish_launch(0);
        configured[unit][dev] = true;
    }
    const int rows_per_cta = kGemvWarps / SPLIT;
    const int dflt = unit ? (smem > 100 * 1024 ? 1 : 2) : (smem > 100 * 1024 ? 1 : (smem > 56 * 1024 ? 2 : 4));
    const int per_sm = tune("gemv.ctas_per_sm", dflt);
    int grid = (N + rows_per_cta - 1) / rows_per_cta;
    if (grid > kSmCount * per_sm) grid = kSmCount * per_sm;
    const int min_grid = (N + rows_per_cta * kGemvMaxIters - 1) / (rows_per_cta * kGemvMaxIters);   // at most kGemvMaxIters passes
    if (unit && SPLIT > 1 && grid < min_grid) grid = min_grid;
    launch_kernel(kern, grid, kGemvWarps * 32, smem, st, static_cast<const __nv_bfloat16*>(x), static_cast<const uint4*>(W),
                  w_scale, static_cast<__nv_bfloat16*>(y), N, kv);
    return finish_launch(1);
}

}  // namespace nmt

extern "C" {

int nmt_gemv_w8a16(const void* x_bf16, const void* W_e4m3, const float* w_scale, void* y_bf16, int64_t N, int64_t K,
                   void* stream) {
    using namespace nmt;
    if (N < 0 || K <= 0 || (K % 16) != 0 || N > 0x7fffffff) return NMT_ERR_SHAPE;
    if (N == 0) return NMT_OK;
    if (!x_bf16 || !W_e4m3 || !w_scale || !y_bf16) return NMT_ERR_NULL;
    if (!aligned4(x_bf16) || !aligned16(W_e4m3) || !aligned4(w_scale) || (reinterpret_cast<uintptr_t>(y_bf16) & 1u)) return NMT_ERR_ALIGN;
    if (K > 45000) return NMT_ERR_UNSUPPORTED;                        // x must fit shared memory as fp32
    const int kv = static_cast<int>(K / 16);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // K-slices of roughly 3 KB: 1 up to K = 4096, 2 up to 8192, 4 up to 16384, 8 beyond.
    int split = tune("gemv.split", K <= 4096 ? 1 : (K <= 8192 ? 2 : (K <= 16384 ? 4 : 8)));
    if (split >= 8) return launch_gemv<8>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    if (split >= 4) return launch_gemv<4>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    if (split >= 2) return launch_gemv<2>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    return launch_gemv<1>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
}

}  // extern "C"
