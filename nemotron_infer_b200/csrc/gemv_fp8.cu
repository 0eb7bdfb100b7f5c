// W8A16 GEMV for single-token decode: y[n] = (sum_k e4m3(W[n,k]) * bf16(x[k])) * w_scale[n].
//
// With one token the projection is pure weight streaming (24-55 MB of e4m3 per matrix, 5.4 GB per token for the
// whole model, ops/gemv.cuh:4-6): the only thing that matters is how fast W crosses HBM, and a matrix is gone in
// a few microseconds, so every SM has to have deep loads in flight from its first cycle.
//
// Kernels, in the order of the file: two CUDA-core kernels (the general fallback: any K that is a multiple of 16, exact
// fp32 products for every x; "gemv.variant" = 1 / 2), the register-streaming tensor-core kernel
// (gemv_w8a16_mma_kernel, the default: K % 64 == 0, f16 MMA after converting the weights).  Common to all:
//   * Persistent grid.  x is converted once per CTA into shared memory.
//   * A work unit is (rows, K-slice): rows are cut into slices of a few KB so that short-and-wide matrices
//     (down_proj: 3136 rows of 12544) still give every warp several units; the warps that share a row sit
//     in one CTA and combine their partial sums through shared memory in a fixed order (deterministic).
//   * fp32 accumulation throughout -- the arithmetic the reference specifies (ops/gemv.cuh:20-22), no fp16 accumulation.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "nmt_common.cuh"

namespace nmt {

constexpr int kGemvWarps = 8;
constexpr int kDefaultGemvVariant = 3;    // 5 = tcgen05 + TMA (gemv_umma.cu), 3 = mma.sync inner product, 1 / 2 = CUDA-core kernels

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

// ---------------------------------------------------------------------------------------------
// Tensor-core inner product.  The CUDA-core kernels above spend ~2.8 instructions per weight byte (convert,
// convert, multiply-add) and are bound by instruction issue at ~3 TB/s.  mma.sync.m16n8k16 (f16 in, fp32
// accumulate) does the multiply-adds and the f16 -> fp32 widening in one instruction per 256 weights per warp,
// leaving one e4m3x2 -> f16x2 convert per two weights.
//
// A dot product does not care in which order k is visited as long as W and x agree, so a lane feeds the MMA
// straight from the 16 contiguous weight bytes it loaded (no shuffles): in chunk c (64 values of k), lane
// (g = lane / 4, t = lane % 4) holds bytes [t*16, t*16+16) of A-rows g and g+8, and MMA m of the chunk uses bytes
// 4m..4m+3 of them; the x fragment is read with the same permutation.
//
// The 16 A-rows of a warp tile are R matrix rows x S "k-streams" (R * S = 16): stream s of a row is multiplied
// with column s of B, which holds x for that stream's k range, so C[s*R + r][s] is a partial sum of matrix row r.
// Together with SPLIT warps per tile this cuts every row into S * SPLIT slices of ~6 chunks, which gives short,
// wide matrices (down_proj: 3136 x 12544) as many work units as tall ones.  All partial sums of a row meet in
// shared memory and are added in a fixed order after one block barrier.
//
// x is staged as f16 scaled by a power of two chosen from max|x| (bf16 has 8 significant bits, f16 has 11, so
// the conversion is exact for every element within 2^-28 of the maximum); the scale is undone on the fp32 sum.
// ---------------------------------------------------------------------------------------------
constexpr int kMmaGroup = 4;          // chunks (64 k each) per load group; two groups are in flight per warp
constexpr int kMmaMaxChunks = 16;     // upper bound on chunks per work unit (keeps the slice count meaningful)

// Bytes 0-1 / bytes 2-3 of a word of four e4m3 weights as an f16x2 register.
__device__ __forceinline__ uint32_t e4m3_lo(uint32_t w) {
    uint32_t h;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, lo; }" : "=r"(h) : "r"(w));
    return h;
}
__device__ __forceinline__ uint32_t e4m3_hi(uint32_t w) {
    uint32_t h;
    asm("{ .reg .b16 lo, hi; mov.b32 {lo, hi}, %1; cvt.rn.f16x2.e4m3x2 %0, hi; }" : "=r"(h) : "r"(w));
    return h;
}
// 16-byte streaming load that is skipped (v keeps its value) when on is false.
__device__ __forceinline__ void ld_stream_if(uint4& v, const void* p, bool on) {
    asm volatile("{ .reg .pred q; setp.ne.s32 q, %5, 0; @q ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4]; }"
                 : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w) : "l"(p), "r"(static_cast<int>(on)) : "memory");
}
// Shared memory for x as f16 (K is a multiple of 64) followed by one chunk of zeros.
__host__ __device__ constexpr size_t mma_x_bytes(int K) { return (size_t)K * 2 + 128; }
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What a decode block does around its projections, folded into the GEMV: the pre-norm RMSNorm of the hidden state
// in front (model/mlp_block.cuh:140, model/mamba_block.cuh:473), relu^2 (model/mlp_block.cuh:145-147) and the
// residual add (model/mlp_block.cuh:170-172, model/mamba_block.cuh:512-514) behind.  Every CTA needs all of x
// anyway, so each one normalises its own copy; the arithmetic and the order of the partial sums are those of the
// stand-alone kernels, so the fused result is byte-identical to "norm kernel, GEMV, activation kernel, add kernel".
struct GemvFusion {
    const float* norm_w;          // non-null: x = rmsnorm(x) * norm_w first
    float eps, inv_cols;
    int norm_threads;             // threads per row of the stand-alone norm kernel (its summation order)
    int activation;               // 1: y = relu(y)^2
    const uint16_t* residual;     // non-null: y += residual[row]
    const uint4* gate;            // non-null: x = gated_rmsnorm(x, gate) * norm_w over groups of group_vecs * 8 columns
    int group_vecs;               // 16-byte vectors per group
    float inv_group;              // 1 / columns per group
    // non-null conv_state: output rows [conv_lo, conv_lo + conv_dim) are channels of Mamba-2's causal conv; instead of being
    // stored they go through the single-token conv step (window in conv_state [conv_dim][3] fp32, updated in place) and
    // SiLU, and land in the x | B | C tensors conv_out[0..2] of conv_n0 / conv_n1 / the remaining channels
    float* conv_state;
    const float* conv_w;          // [conv_dim][4]
    const float* conv_bias;       // [conv_dim]
    uint16_t* conv_out[3];
    int conv_lo, conv_dim, conv_n0, conv_n1;
};

// ---------------------------------------------------------------------------------------------
// Staging of x.  Every CTA needs all of x in shared memory in the MMA's operand format, and (fused form) normalises
// its own copy first.  This runs once per CTA and sits between the kernel's start
// and its first MMA, so its length is a fixed cost of every launch: the loops below are bounded by K (8 bf16 per
// thread and step, 16-byte accesses) - an earlier version walked a fully unrolled 32-slot register array whatever K
// was and spent ~900 warp instructions per warp on a 3136-wide x, a third of the kernel's instruction stream.
//   1. optional RMSNorm in the stand-alone kernel's shape (rmsnorm_ctarow_kernel, one row): norm_threads threads,
//      thread t owns vectors t, t + norm_threads, ...; per-thread f32x2 sums, warp shuffle, then the warps in order -
//      the normalised bf16 row lands in `xn` (shared memory) and equals the stand-alone kernel's output bit for bit;
//   2. max|x| -> exponent e so that max|x| * 2^-e lies in [2^14, 2^15);
//   3. x * 2^-e -> f16, plus one chunk of zeros.
// Returns e.  Ends with a block barrier; all kGemvWarps * 32 threads must call it.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int stage_x(const __nv_bfloat16* __restrict__ x, const GemvFusion& fu, int K, uint8_t* xs, uint4* xn,
                                       float* s_red) {
    constexpr int NT = kGemvWarps * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nv = K / 8;                                          // 16-byte vectors of x
    const uint4* xv = reinterpret_cast<const uint4*>(x);
    const bool normed = fu.norm_w != nullptr;                      // block-uniform
    if (normed && fu.gate) {
        // The Mamba-2 gated norm in the stand-alone kernel's shape (gated_groupwarp_kernel): one warp per group, lane l
        // owns vectors l, l + 32, ... of the group, per-lane f32x2 sums in that order, one butterfly - the normalised
        // bf16 row equals the stand-alone kernel's output bit for bit.  g is recomputed in the second walk instead of
        // being kept in registers (the weight stream's first two load groups live there at this point).
        const int gv = fu.group_vecs, ngroups = nv / gv;
        for (int grp = warp; grp < ngroups; grp += kGemvWarps) {
            const uint4* yg = xv + (size_t)grp * gv;
            const uint4* zg = fu.gate + (size_t)grp * gv;
            float2 acc = make_float2(0.f, 0.f);
            for (int v = lane; v < gv; v += 32) {
                float2 py[4], pz[4];
                unpack8x2(ld_stream(yg + v), py);
                unpack8x2(ld_stream(zg + v), pz);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 g = __fmul2_rn(py[k], silu2_sfu(pz[k]));
                    acc = __ffma2_rn(g, g, acc);
                }
            }
            const float ss = warp_sum(acc.x + acc.y);
            const float rstd = rsqrtf(ss * fu.inv_group + fu.eps);
            const float* wg = fu.norm_w + (size_t)grp * gv * 8;
            for (int v = lane; v < gv; v += 32) {
                float2 py[4], pz[4], g[4];
                unpack8x2(ld_stream(yg + v), py);
                unpack8x2(ld_stream(zg + v), pz);
#pragma unroll
                for (int k = 0; k < 4; ++k) g[k] = __fmul2_rn(py[k], silu2_sfu(pz[k]));
                xn[(size_t)grp * gv + v] = scale8(g, rstd, ld_weight4(wg + v * 8), ld_weight4(wg + v * 8 + 4));
            }
        }
        __syncthreads();
    } else if (normed) {
        const int nt = fu.norm_threads;
        if (threadIdx.x < nt) {
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll 2
            for (int v = threadIdx.x; v < nv; v += nt) {
                float2 pr[4];
                unpack8x2(ld_stream(xv + v), pr);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc = __ffma2_rn(pr[k], pr[k], acc);
            }
            const float ss = warp_sum(acc.x + acc.y);
            if (lane == 0) s_red[warp] = ss;
        }
        __syncthreads();
        if (threadIdx.x < nt) {
            float total = 0.f;
            for (int i = 0; i < nt / 32; ++i) total += s_red[i];
            const float rstd = rsqrtf(total * fu.inv_cols + fu.eps);
#pragma unroll 2
            for (int v = threadIdx.x; v < nv; v += nt) {
                float2 pr[4];
                unpack8x2(ld_stream(xv + v), pr);                  // second read of a row that sits in L1 / L2
                xn[v] = scale8(pr, rstd, ld_weight4(fu.norm_w + (size_t)v * 8), ld_weight4(fu.norm_w + (size_t)v * 8 + 4));
            }
        }
        __syncthreads();
    }
    const uint4* src = normed ? xn : xv;
    float m = 0.f;
#pragma unroll 2
    for (int v = threadIdx.x; v < nv; v += NT) {
        const uint4 u = normed ? src[v] : __ldg(src + v);
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) m = fmaxf(m, fmaxf(fabsf(bf16_lo(w4[k])), fabsf(bf16_hi(w4[k]))));
    }
    m = warp_max(m);
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    float mm = 0.f;
#pragma unroll
    for (int i = 0; i < kGemvWarps; ++i) mm = fmaxf(mm, s_red[i]);
    int e = 0;
    if (mm > 0.f && mm < 3.0e38f) e = static_cast<int>((__float_as_uint(mm) >> 23) & 0xff) - 127 - 14;   // max|x| lands in [2^14, 2^15)
    e = max(e, -100);                                              // keeps 2^-e and 2^e normal fp32 numbers
    const float down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);      // 2^-e
#pragma unroll 2
    for (int v = threadIdx.x; v < nv; v += NT) {
        const uint4 u = normed ? src[v] : __ldg(src + v);
        const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
        uint32_t hw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            __half2 h2 = __floats2half2_rn(bf16_lo(w4[k]) * down, bf16_hi(w4[k]) * down);
            hw[k] = *reinterpret_cast<uint32_t*>(&h2);
        }
        *reinterpret_cast<uint4*>(xs + (size_t)v * 16) = make_uint4(hw[0], hw[1], hw[2], hw[3]);
    }
    // one chunk of zeros behind x: what lanes with nothing to contribute multiply with
    uint8_t* zero = xs + (size_t)K * 2;
    if (threadIdx.x < 32) reinterpret_cast<uint32_t*>(zero)[threadIdx.x] = 0u;
    __syncthreads();
    return e;
}

// Two CTAs per SM are part of the design (16 warps keep the convert-and-multiply stream issuing): the bound makes the
// compiler hold the kernel at 128 registers instead of silently taking more and halving the occupancy (measured once by
// accident: 12.7 us instead of 9.0).
template <int SPLIT, int S>           // S k-streams per tile, R = 16 / S matrix rows per tile
__global__ void __launch_bounds__(kGemvWarps * 32, 2)
gemv_w8a16_mma_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ W, const float* __restrict__ w_scale,
                      __nv_bfloat16* __restrict__ y, int N, int K, int iters, int early_trigger, GemvFusion fu) {
    constexpr int R = 16 / S;
    constexpr int TILES_PER_CTA = kGemvWarps / SPLIT;
    constexpr int Q = S * SPLIT;                                   // k-slices per matrix row
    constexpr int G = kMmaGroup;                                   // chunks per load group
    extern __shared__ __align__(16) uint8_t smem_b[];
    __half* xh = reinterpret_cast<__half*>(smem_b);                // K halves
    float* part = reinterpret_cast<float*>(smem_b + mma_x_bytes(K));                   // [iters][warp][16]
    __shared__ float s_red[kGemvWarps];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- this warp's slice geometry ----
    const int kc = K / 64;                                         // chunks per row
    // Slice q gets base chunks, the LAST rem slices one more: a short slice that reads one chunk past its end (to
    // keep the loop uniform) then reads the first chunk of the next slice of the same row, which is inside the matrix.
    const int base = kc / Q, rem = kc % Q;
    auto slice_start = [&](int q) { return q * base + max(0, q - (Q - rem)); };
    auto slice_len = [&](int q) { return base + (q >= Q - rem ? 1 : 0); };
    const int split_id = warp % SPLIT, tile_in_cta = warp / SPLIT;
    // A-rows of this lane: a = g and a = g + 8; stream = a / R, local row = a % R
    const int sA = g / R, rA = g % R, sB = (g + 8) / R, rB = (g + 8) % R;
    const int cA0 = slice_start(split_id * S + sA), cB0 = slice_start(split_id * S + sB);
    // x fragment: lanes with g < S feed column g of B with stream g's k range
    const int cX0 = g < S ? slice_start(split_id * S + g) : 0, nX = g < S ? slice_len(split_id * S + g) : 0;
    const int nmax = base + (rem ? 1 : 0);
    const int groups = (nmax + G - 1) / G;                         // load groups per work unit
    const int ntiles = (N + R - 1) / R;

    // Ragged edges are handled on the x side so that no weight register ever needs a zero fill: a row past N is read
    // from row N-1 (its sum is never stored), a chunk past the end of a short stream is the next stream's first
    // chunk (inside the matrix) and is multiplied with zeros, because lanes that have no x to contribute for a
    // chunk (g >= S, or past their stream's end) read the zero block that follows x in shared memory.
    const __half* xzero = xh + K;                                  // 64 halves of zero
    const __half* xbase = xh + (size_t)cX0 * 64 + t * 16;
    const size_t offA = (size_t)cA0 * 64 + t * 16, offB = (size_t)cB0 * 64 + t * 16;

    // Load group (it, grp) = chunks [grp*G, grp*G + G) of work unit it, for both A-rows of this lane.
    auto load_group = [&](uint4 (&wa)[G], uint4 (&wb)[G], int it, int grp) {
        // Predicated loads, not branches: a branch around loads makes the compiler wait for them at the join.
        const int tile = (it * gridDim.x + blockIdx.x) * TILES_PER_CTA + tile_in_cta;
        const bool live = it < iters && tile < ntiles;             // warp-uniform
        const int j0 = grp * G;
        const int tl = min(tile, ntiles - 1);
        const uint8_t* pa = W + (size_t)min(tl * R + rA, N - 1) * K + offA + j0 * 64;
        const uint8_t* pb = W + (size_t)min(tl * R + rB, N - 1) * K + offB + j0 * 64;
#pragma unroll
        for (int j = 0; j < G; ++j) {
            const bool on = live && j0 + j < nmax;
            ld_stream_if(wa[j], pa + j * 64, on);
            ld_stream_if(wb[j], pb + j * 64, on);
        }
    };
    float c[4] = {0.f, 0.f, 0.f, 0.f}, d[4] = {0.f, 0.f, 0.f, 0.f};    // two chains, so an MMA does not wait for the one before it
    auto compute_group = [&](const uint4 (&wa)[G], const uint4 (&wb)[G], int it, int grp) {
        const int tile = (it * gridDim.x + blockIdx.x) * TILES_PER_CTA + tile_in_cta;
        if (it >= iters) return;                                   // warp-uniform
        if (tile < ntiles) {
            const int j0 = grp * G;
            if (grp == 0) c[0] = c[1] = c[2] = c[3] = d[0] = d[1] = d[2] = d[3] = 0.f;
#pragma unroll
            for (int j = 0; j < G; ++j) {
                if (j0 + j < nmax) {                               // warp-uniform
                    const uint4* xp = reinterpret_cast<const uint4*>(j0 + j < nX ? xbase + (j0 + j) * 64 : xzero);
                    const uint4 x0 = xp[0], x1 = xp[1];
                    const uint32_t wa_[4] = {wa[j].x, wa[j].y, wa[j].z, wa[j].w};
                    const uint32_t wb_[4] = {wb[j].x, wb[j].y, wb[j].z, wb[j].w};
                    const uint32_t xb_[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int mm = 0; mm < 4; ++mm)
                        mma_f16((mm & 1) ? d : c, e4m3_lo(wa_[mm]), e4m3_lo(wb_[mm]), e4m3_hi(wa_[mm]), e4m3_hi(wb_[mm]), xb_[2 * mm], xb_[2 * mm + 1]);
                }
            }
        }
        if (grp == groups - 1) {
            // C[a][n] is wanted for n = stream(a) only: lane (g, t) holds columns 2t, 2t+1 of A-rows g and g+8
            float* pw = part + ((size_t)it * kGemvWarps + warp) * 16;
            if (sA / 2 == t) pw[g] = (sA & 1) ? c[1] + d[1] : c[0] + d[0];
            if (sB / 2 == t) pw[g + 8] = (sB & 1) ? c[3] + d[3] : c[2] + d[2];
        }
    };

    // The weights are constants of the model, not an output of the preceding kernel: the first two load groups go out
    // before the wait on that kernel, and before x is staged, so the stream is already running when x is ready.
    uint4 wa0[G] = {}, wb0[G] = {}, wa1[G] = {}, wb1[G] = {};
    int cit = 0, cgrp = 0, lit = 0, lgrp = 0;                      // (work unit, group) being computed / loaded
    auto step = [&](int& it, int& grp) { if (++grp == groups) { grp = 0; ++it; } };
    load_group(wa0, wb0, lit, lgrp);
    step(lit, lgrp);
    load_group(wa1, wb1, lit, lgrp);
    step(lit, lgrp);
    pdl_wait();

    uint4* xn = reinterpret_cast<uint4*>(part + (size_t)iters * kGemvWarps * 16);        // K bf16: the normalised x
    const int e = stage_x(x, fu, K, reinterpret_cast<uint8_t*>(xh), xn, s_red);

    // What the epilogue needs from global memory for this thread's first output row (its only one unless a CTA makes more
    // than 256 / 16 passes) is requested now, so that it is not a dependent load at the very end of the kernel.
    float first_scale = 0.f;
    uint32_t first_res = 0u;
    {
        const int o = threadIdx.x;
        if (o < iters * TILES_PER_CTA * R) {
            const int it = o / (TILES_PER_CTA * R), rest = o % (TILES_PER_CTA * R);
            const int row = ((it * gridDim.x + blockIdx.x) * TILES_PER_CTA + rest / R) * R + rest % R;
            if (row < N) {
                first_scale = __ldg(w_scale + row);
                if (fu.residual) first_res = fu.residual[row];
            }
        }
    }

    // ---- stream: the next groups' loads are in flight while this group is multiplied ----
#pragma unroll 1
    while (cit < iters) {
        compute_group(wa0, wb0, cit, cgrp);
        step(cit, cgrp);
        load_group(wa0, wb0, lit, lgrp);
        step(lit, lgrp);
        compute_group(wa1, wb1, cit, cgrp);
        step(cit, cgrp);
        load_group(wa1, wb1, lit, lgrp);
        step(lit, lgrp);
        if (early_trigger && lit >= iters) pdl_trigger();          // every load of this warp has been issued
    }
    __syncthreads();
    // ---- combine: matrix row r of tile T = sum over streams s and split warps of part[..][s*R + r] ----
    const float up = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);         // 2^e
    for (int o = threadIdx.x; o < iters * TILES_PER_CTA * R; o += blockDim.x) {
        const int it = o / (TILES_PER_CTA * R), rest = o % (TILES_PER_CTA * R);
        const int tc = rest / R, r = rest % R;
        const int row = ((it * gridDim.x + blockIdx.x) * TILES_PER_CTA + tc) * R + r;
        if (row < N) {
            float sum = 0.f;
#pragma unroll
            for (int sp = 0; sp < SPLIT; ++sp)
#pragma unroll
                for (int s2 = 0; s2 < S; ++s2) sum += part[((size_t)it * kGemvWarps + tc * SPLIT + sp) * 16 + s2 * R + r];
            // bf16 result in the low half of a pair, so the epilogues can use the stand-alone kernels' instructions
            const bool first = o == static_cast<int>(threadIdx.x);
            uint32_t yb = pack_bf16x2((sum * up) * (first ? first_scale : __ldg(w_scale + row)), 0.f);
            if (fu.activation == 1) yb = relu2_bf16x2(yb);
            if (fu.residual) yb = add_bf16x2_rn(first ? first_res : static_cast<uint32_t>(fu.residual[row]), yb);
            const int ch = row - fu.conv_lo;
            if (fu.conv_state && ch >= 0 && ch < fu.conv_dim) {
                // the conv step of this channel, in the stand-alone kernel's arithmetic (conv1d_silu_decode_split_kernel):
                // bias, then taps oldest to newest, the bf16-rounded projection as the newest input
                const float xin = bf16_lo(yb);
                float* sp = fu.conv_state + (size_t)ch * 3;
                const float s0 = sp[0], s1 = sp[1], s2 = sp[2];
                const float4 wt = ld_weight4(fu.conv_w + (size_t)ch * 4);
                float acc = __ldg(fu.conv_bias + ch);
                acc = fmaf(wt.x, s0, acc);
                acc = fmaf(wt.y, s1, acc);
                acc = fmaf(wt.z, s2, acc);
                acc = fmaf(wt.w, xin, acc);
                sp[0] = s1;
                sp[1] = s2;
                sp[2] = xin;
                int col = ch, seg = 0;
                if (col >= fu.conv_n0) { col -= fu.conv_n0; seg = 1; if (col >= fu.conv_n1) { col -= fu.conv_n1; seg = 2; } }
                uint16_t* dst = seg == 0 ? fu.conv_out[0] : seg == 1 ? fu.conv_out[1] : fu.conv_out[2];
                dst[col] = static_cast<uint16_t>(pack_bf16x2(silu_sfu(acc), 0.f) & 0xffffu);
            } else {
                reinterpret_cast<uint16_t*>(y)[row] = static_cast<uint16_t>(yb & 0xffffu);
            }
        }
    }
    if (!early_trigger) pdl_trigger();
}

template <int SPLIT, int S>
static int launch_gemv_mma(const void* x, const void* W, const float* w_scale, void* y, int N, int K, const GemvFusion& fu, cudaStream_t st) {
    constexpr int R = 16 / S, TILES_PER_CTA = kGemvWarps / SPLIT;
    auto kern = gemv_w8a16_mma_kernel<SPLIT, S>;
    const int ntiles = (N + R - 1) / R;
    const int ctas_needed = (ntiles + TILES_PER_CTA - 1) / TILES_PER_CTA;
    // Every SM gets its full complement of CTAs and the work units go round them (unit u belongs to CTA u % grid), so
    // that no SM carries more than one unit more than another: with the grid shrunk to ceil(units / passes) some SMs
    // held two CTAs and some one, and the busiest SM had 13 % more bytes than the average at the model's shapes.
    const int per_sm = tune("gemv.ctas_per_sm", 2);
    const int grid = ctas_needed < kSmCount * per_sm ? ctas_needed : kSmCount * per_sm;
    const int iters = (ctas_needed + grid - 1) / grid;                            // passes of the busiest CTA
    const size_t smem = mma_x_bytes(K) + (size_t)iters * kGemvWarps * 16 * sizeof(float) + (fu.norm_w ? (size_t)K * 2 : 0);
    if (smem > 200 * 1024) return NMT_ERR_UNSUPPORTED;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return finish_launch(0);
        configured[dev] = true;
    }
    launch_kernel(kern, grid, kGemvWarps * 32, smem, st, static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(W),
                  w_scale, static_cast<__nv_bfloat16*>(y), N, K, iters, tune("gemv.early_trigger", 1) == 1, fu);
    return finish_launch(1);
}

// Picks S * SPLIT so that a work unit is about six chunks; returns NMT_ERR_UNSUPPORTED when the shape does not fit.
static int launch_gemv_mma_auto(const void* x, const void* W, const float* w_scale, void* y, int N, int K, const GemvFusion& fu, cudaStream_t st) {
    if ((K % 64) != 0) return NMT_ERR_UNSUPPORTED;
    const int kc = K / 64;
    int q = 1;
    while (q < 64 && (kc + q - 1) / q > tune("gemv.unit_chunks", 7)) q *= 2;                                 // slices per row
    if ((kc + q - 1) / q > kMmaMaxChunks) return NMT_ERR_UNSUPPORTED;
    const int forced = tune("gemv.streams", 0);
    int split = q >= 8 ? 8 : q, streams = q / split;
    if (forced > 0 && forced <= 8 && q % forced == 0 && q / forced <= 8) { streams = forced; split = q / forced; }
#define NMT_MMA_CASE(SP, ST) if (split == SP && streams == ST) return launch_gemv_mma<SP, ST>(x, W, w_scale, y, N, K, fu, st)
    NMT_MMA_CASE(1, 1); NMT_MMA_CASE(2, 1); NMT_MMA_CASE(4, 1); NMT_MMA_CASE(8, 1);
    NMT_MMA_CASE(1, 2); NMT_MMA_CASE(2, 2); NMT_MMA_CASE(4, 2); NMT_MMA_CASE(8, 2);
    NMT_MMA_CASE(1, 4); NMT_MMA_CASE(2, 4); NMT_MMA_CASE(4, 4); NMT_MMA_CASE(8, 4);
    NMT_MMA_CASE(1, 8); NMT_MMA_CASE(2, 8); NMT_MMA_CASE(4, 8); NMT_MMA_CASE(8, 8);
#undef NMT_MMA_CASE
    return NMT_ERR_UNSUPPORTED;
}

int launch_gemv_umma(const void* x, const float* norm_w, float eps, const void* W, const float* w_scale, int activation,
                     const void* residual, void* y, int N, int K, cudaStream_t st);      // gemv_umma.cu

template <int SPLIT>
static int launch_gemv(const void* x, const void* W, const float* w_scale, void* y, int N, int kv, cudaStream_t st) {
    constexpr int UNROLL = 4;
    const bool unit = (kv + SPLIT - 1) / SPLIT <= kGemvSlots * 32 && tune("gemv.variant", 1) != 2;
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

int nmt_gemv_w8a16_fused(const void* x_bf16, const float* norm_w, float eps, const void* W_e4m3, const float* w_scale,
                         int activation, const void* residual_bf16, void* y_bf16, int64_t N, int64_t K, void* stream) {
    using namespace nmt;
    if (N < 0 || K <= 0 || (K % 16) != 0 || N > 0x7fffffff || activation < 0 || activation > 1) return NMT_ERR_SHAPE;
    if (N == 0) return NMT_OK;
    if (!x_bf16 || !W_e4m3 || !w_scale || !y_bf16) return NMT_ERR_NULL;
    if (!aligned4(x_bf16) || !aligned16(W_e4m3) || !aligned4(w_scale) || (reinterpret_cast<uintptr_t>(y_bf16) & 1u) ||
        (norm_w && (!aligned16(x_bf16) || !aligned16(norm_w))) || (reinterpret_cast<uintptr_t>(residual_bf16) & 1u))
        return NMT_ERR_ALIGN;
    GemvFusion fu = {};
    fu.norm_w = norm_w;
    fu.eps = eps;
    fu.inv_cols = 1.0f / static_cast<float>(K);
    fu.norm_threads = default_norm_block(K / 8, false);
    fu.activation = activation;
    fu.residual = static_cast<const uint16_t*>(residual_bf16);
    // The prologue keeps a thread's share of x in 8 registers-vectors; the fused forms exist only on the tensor-core kernel.
    if (norm_w && (fu.norm_threads > kGemvWarps * 32 || (K / 8 + fu.norm_threads - 1) / fu.norm_threads > 8)) return NMT_ERR_UNSUPPORTED;
    if (tune("gemv.variant", kDefaultGemvVariant) == 5) {
        const int r = launch_gemv_umma(x_bf16, norm_w, eps, W_e4m3, w_scale, activation, residual_bf16, y_bf16, static_cast<int>(N),
                                       static_cast<int>(K), static_cast<cudaStream_t>(stream));
        if (r != NMT_ERR_UNSUPPORTED) return r;
    }
    return launch_gemv_mma_auto(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), static_cast<int>(K), fu,
                                static_cast<cudaStream_t>(stream));
}

int nmt_gemv_w8a16_fused_conv_step(const void* x_bf16, const float* norm_w, float eps, const void* W_e4m3, const float* w_scale,
                                   void* y_bf16, int64_t N, int64_t K, int64_t conv_row_lo, const float* conv_w,
                                   const float* conv_bias, float* conv_state, void* out0, void* out1, void* out2, int64_t n0,
                                   int64_t n1, int64_t n2, void* stream) {
    using namespace nmt;
    if (N < 0 || K <= 0 || (K % 64) != 0 || N > 0x7fffffff || n0 < 0 || n1 < 0 || n2 < 0 || conv_row_lo < 0 ||
        conv_row_lo + n0 + n1 + n2 > N)
        return NMT_ERR_SHAPE;
    if (N == 0) return NMT_OK;
    const int64_t conv_dim = n0 + n1 + n2;
    if (!x_bf16 || !W_e4m3 || !w_scale || !y_bf16 || (conv_dim > 0 && (!conv_w || !conv_bias || !conv_state)) || (n0 > 0 && !out0) ||
        (n1 > 0 && !out1) || (n2 > 0 && !out2))
        return NMT_ERR_NULL;
    auto odd = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) != 0; };
    if (!aligned4(x_bf16) || !aligned16(W_e4m3) || !aligned4(w_scale) || odd(y_bf16) || odd(out0) || odd(out1) || odd(out2) ||
        (norm_w && (!aligned16(x_bf16) || !aligned16(norm_w))) || !aligned16(conv_w) || !aligned4(conv_bias) || !aligned4(conv_state))
        return NMT_ERR_ALIGN;
    GemvFusion fu = {};
    fu.norm_w = norm_w;
    fu.eps = eps;
    fu.inv_cols = 1.0f / static_cast<float>(K);
    fu.norm_threads = default_norm_block(K / 8, false);
    if (norm_w && (K > 10240 || fu.norm_threads > kGemvWarps * 32 || (K / 8 + fu.norm_threads - 1) / fu.norm_threads > 8)) return NMT_ERR_UNSUPPORTED;
    if (conv_dim > 0) {
        fu.conv_state = conv_state;
        fu.conv_w = conv_w;
        fu.conv_bias = conv_bias;
        fu.conv_out[0] = static_cast<uint16_t*>(out0);
        fu.conv_out[1] = static_cast<uint16_t*>(out1);
        fu.conv_out[2] = static_cast<uint16_t*>(out2);
        fu.conv_lo = static_cast<int>(conv_row_lo);
        fu.conv_dim = static_cast<int>(conv_dim);
        fu.conv_n0 = static_cast<int>(n0);
        fu.conv_n1 = static_cast<int>(n1);
    }
    return launch_gemv_mma_auto(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), static_cast<int>(K), fu,
                                static_cast<cudaStream_t>(stream));
}

int nmt_gemv_w8a16_gated(const void* y_in_bf16, const void* gate_bf16, const float* gnorm_w, float eps, int64_t group_size,
                         const void* W_e4m3, const float* w_scale, const void* residual_bf16, void* out_bf16, int64_t N, int64_t K,
                         void* stream) {
    using namespace nmt;
    if (N < 0 || K <= 0 || (K % 64) != 0 || N > 0x7fffffff || group_size <= 0 || (group_size % 8) != 0 || (K % group_size) != 0)
        return NMT_ERR_SHAPE;
    if (N == 0) return NMT_OK;
    if (!y_in_bf16 || !gate_bf16 || !gnorm_w || !W_e4m3 || !w_scale || !out_bf16) return NMT_ERR_NULL;
    if (!aligned16(y_in_bf16) || !aligned16(gate_bf16) || !aligned16(gnorm_w) || !aligned16(W_e4m3) || !aligned4(w_scale) ||
        (reinterpret_cast<uintptr_t>(out_bf16) & 1u) || (reinterpret_cast<uintptr_t>(residual_bf16) & 1u))
        return NMT_ERR_ALIGN;
    // the normalised row lives in shared memory beside x; groups wider than 2048 take another stand-alone kernel
    if (K > 10240 || group_size > 2048) return NMT_ERR_UNSUPPORTED;
    GemvFusion fu = {};
    fu.norm_w = gnorm_w;
    fu.eps = eps;
    fu.gate = static_cast<const uint4*>(gate_bf16);
    fu.group_vecs = static_cast<int>(group_size / 8);
    fu.inv_group = 1.0f / static_cast<float>(group_size);
    fu.residual = static_cast<const uint16_t*>(residual_bf16);
    return launch_gemv_mma_auto(y_in_bf16, W_e4m3, w_scale, out_bf16, static_cast<int>(N), static_cast<int>(K), fu,
                                static_cast<cudaStream_t>(stream));
}

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
    const int variant = tune("gemv.variant", kDefaultGemvVariant);
    if (variant == 5) {
        const int r = launch_gemv_umma(x_bf16, nullptr, 0.f, W_e4m3, w_scale, 0, nullptr, y_bf16, static_cast<int>(N), static_cast<int>(K), st);
        if (r != NMT_ERR_UNSUPPORTED) return r;
    }
    if (variant >= 3) {
        const int r = launch_gemv_mma_auto(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), static_cast<int>(K), GemvFusion{}, st);
        if (r != NMT_ERR_UNSUPPORTED) return r;
    }
    // K-slices of roughly 3 KB: 1 up to K = 4096, 2 up to 8192, 4 up to 16384, 8 beyond.
    int split = tune("gemv.split", K <= 4096 ? 1 : (K <= 8192 ? 2 : (K <= 16384 ? 4 : 8)));
    if (split >= 8) return launch_gemv<8>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    if (split >= 4) return launch_gemv<4>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    if (split >= 2) return launch_gemv<2>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
    return launch_gemv<1>(x_bf16, W_e4m3, w_scale, y_bf16, static_cast<int>(N), kv, st);
}

}  // extern "C"
