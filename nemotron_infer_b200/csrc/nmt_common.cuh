// Shared device helpers and host-side argument checks for the sm_100a kernels.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <atomic>

#include "nemotron_b200.h"

namespace nmt {

constexpr int kSmCount = 148;   // B200: 2 dies x 74 SMs

// ---------------------------------------------------------------------------
// 128-bit global memory access.  Activations are touched once, so loads skip L1
// allocation (leaving L1 for the fp32 weight vector, which every row re-reads).
// Plain (coherent) loads, not .nc: several entry points allow in-place use.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream(uint4* p, const uint4& v) {
    asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// Read-only data that IS reused (norm weights): cached load.
__device__ __forceinline__ float4 ld_weight4(const float* p) {
    return __ldg(reinterpret_cast<const float4*>(p));
}

// ---------------------------------------------------------------------------
// bf16 <-> fp32 on packed pairs.  A bf16 is the upper half of an fp32, so the
// upcast is a shift / mask; the downcast is cvt.rn.bf16x2.f32 (round to nearest
// even), the same rounding torch applies.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    v.x = pack_bf16x2(f[0], f[1]);
    v.y = pack_bf16x2(f[2], f[3]);
    v.z = pack_bf16x2(f[4], f[5]);
    v.w = pack_bf16x2(f[6], f[7]);
    return v;
}

// ---------------------------------------------------------------------------
// Packed forms.  sm_100 issues fp32 add / mul / fma on register PAIRS (add.rn.f32x2, mul.rn.f32x2,
// fma.rn.f32x2: two IEEE round-to-nearest results per instruction), and bf16 pairs add natively
// (add.bf16x2, one rounding of the exact sum).  Working on the (lo, hi) pair of each 32-bit word halves
// the arithmetic instruction count of these bandwidth-bound kernels without changing a single result bit.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float2 unpack2(uint32_t u) { return make_float2(bf16_lo(u), bf16_hi(u)); }
__device__ __forceinline__ uint32_t pack2(const float2& f) { return pack_bf16x2(f.x, f.y); }
__device__ __forceinline__ void unpack8x2(const uint4& v, float2 (&p)[4]) {
    p[0] = unpack2(v.x); p[1] = unpack2(v.y); p[2] = unpack2(v.z); p[3] = unpack2(v.w);
}
__device__ __forceinline__ uint4 pack8x2(const float2 (&p)[4]) {
    return make_uint4(pack2(p[0]), pack2(p[1]), pack2(p[2]), pack2(p[3]));
}
__device__ __forceinline__ uint32_t add_bf16x2_rn(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("add.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint4 add_bf16x8_rn(const uint4& a, const uint4& b) {
    return make_uint4(add_bf16x2_rn(a.x, b.x), add_bf16x2_rn(a.y, b.y), add_bf16x2_rn(a.z, b.z), add_bf16x2_rn(a.w, b.w));
}
__device__ __forceinline__ uint32_t relu2_bf16x2(uint32_t u) {
    // fma.rn.relu.bf16x2 (x * 1 + 0, clamped at zero): one FMA-pipe instruction per pair; NaN stays NaN
    // and -0 becomes +0.  The reference uses the same instruction (ops/elementwise.cuh:256-268).  The two
    // constants are written as bit patterns: built with a conversion intrinsic they were re-converted on
    // every call and the conversion pipe, not memory, set the pace.
    uint32_t r;
    asm("fma.rn.relu.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(u), "r"(0x3F803F80u), "r"(0u));
    asm("mul.bf16x2 %0, %1, %1;" : "=r"(r) : "r"(r));
    return r;
}
// out = (p * rstd) * w for the eight elements of one vector, in that association order.
__device__ __forceinline__ uint4 scale8(const float2 (&p)[4], float rstd, const float4& w0, const float4& w1) {
    const float2 rs = make_float2(rstd, rstd);
    float2 o[4];
    o[0] = __fmul2_rn(__fmul2_rn(p[0], rs), make_float2(w0.x, w0.y));
    o[1] = __fmul2_rn(__fmul2_rn(p[1], rs), make_float2(w0.z, w0.w));
    o[2] = __fmul2_rn(__fmul2_rn(p[2], rs), make_float2(w1.x, w1.y));
    o[3] = __fmul2_rn(__fmul2_rn(p[3], rs), make_float2(w1.z, w1.w));
    return pack8x2(o);
}

// z / (1 + exp(-z)) through the SFU: 2^(-z*log2 e) and an approximate reciprocal, both good to ~2 ulp of
// fp32, far below the bf16 rounding of the result.  The .ftz forms are single MUFU instructions (the
// denormal-preserving forms expand into range-scaling sequences that made this kernel issue-bound); the only
// visible effect is that silu(z) flushes to zero once |silu(z)| < 2^-126 (z below about -87).
__device__ __forceinline__ float silu_sfu(float z) {
    float e, rcp;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(1.0f + e));
    return z * rcp;
}
// Two at a time: the multiplies and the add run as f32x2 instructions, the two SFU ops stay scalar.
__device__ __forceinline__ float2 silu2_sfu(const float2& z) {
    const float2 t = __fmul2_rn(z, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    float2 e, rcp;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
    const float2 d = __fadd2_rn(e, make_float2(1.0f, 1.0f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp.x) : "f"(d.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp.y) : "f"(d.y));
    return __fmul2_rn(z, rcp);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Non-negative floats order like their bit patterns, so the running maximum is an unsigned atomicMax
// (ops/gemm.cuh:254-255).  Most callers lose the race to an earlier, larger value: peek first.
__device__ __forceinline__ void publish_max(unsigned int* word, float v) {
    const unsigned int bits = __float_as_uint(v);
    if (bits > *reinterpret_cast<volatile unsigned int*>(word)) atomicMax(word, bits);
}
__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Butterfly sum: every lane ends with the warp total.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel first waits until the PREVIOUS kernel in the stream has
// completed and its writes are visible (pdl_wait, before any global access), and as its last act tells the
// scheduler that the NEXT kernel may start launching (pdl_trigger), which hides that kernel's launch
// latency behind this one's last CTAs.  The trigger sits at the END of a CTA's work on purpose: issued at
// the start it let the next kernel's CTAs, parked in their wait, take SM slots from this kernel's own
// not-yet-launched CTAs, and a chain of unlike kernels ran 20 % slower.  Without the launch attribute both
// instructions are no-ops, so the kernels behave identically under a plain launch.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

extern std::atomic<int64_t> g_launches;
int finish_launch(int n_kernels);   // records cudaGetLastError(); returns an nmt_status
int64_t thread_launch_epoch();     // how many calls of this host thread have launched kernels so far
int tune(const char* key, int dflt);  // current value of a tuning knob

bool pdl_enabled();   // runtime.cu: knob "launch.pdl"

// One launch path for every kernel: plain, or with programmatic stream serialization when enabled.
template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(block));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Threads per row of the CTA-per-row norm kernels (and of the statistics pass of the norm + quantiser, which must
// add its partial sums in the same order to stay byte-identical with "norm, then quantise").  Measured from 3136
// to 32,768 columns: about 3 vectors per thread is best with the residual add (6 loads per thread in flight),
// about 5 without it - 3136 columns: 160 / 96 threads (plain norm 6.73 vs 6.24 TB/s for 160 threads x 2 rows),
// 12,544 columns: 512 / 320 threads (plain norm 6.16 vs 4.85 TB/s at 224).  At most 512 threads, so up to 8
// vectors per thread at the 32,768-column limit of these kernels.
inline int default_norm_block(int64_t nv, bool fuse_add) {
    const int per_thread = fuse_add ? 3 : 5;
    int64_t block = (nv + per_thread - 1) / per_thread;
    block = (block + 31) / 32 * 32;
    return block > 512 ? 512 : static_cast<int>(block);
}

// Same, with the grid grouped into thread-block clusters of `cluster` CTAs (grid must be a multiple of it).
template <typename... KArgs, typename... Args>
inline void launch_cluster_kernel(void (*kern)(KArgs...), int grid, int cluster, int block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(static_cast<unsigned>(block));
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

inline int grid_for(int64_t work_items, int items_per_cta, int max_ctas) {
    int64_t g = (work_items + items_per_cta - 1) / items_per_cta;
    if (g < 1) g = 1;
    if (max_ctas > 0 && g > max_ctas) g = max_ctas;
    return static_cast<int>(g);
}

}  // namespace nmt
