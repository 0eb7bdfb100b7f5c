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

// Butterfly sum: every lane ends with the warp total.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

extern std::atomic<int64_t> g_launches;
int finish_launch(int n_kernels);   // records cudaGetLastError(); returns an nmt_status
int tune(const char* key, int dflt);  // current value of a tuning knob

inline int grid_for(int64_t work_items, int items_per_cta, int max_ctas) {
    int64_t g = (work_items + items_per_cta - 1) / items_per_cta;
    if (g < 1) g = 1;
    if (max_ctas > 0 && g > max_ctas) g = max_ctas;
    return static_cast<int>(g);
}

}  // namespace nmt
