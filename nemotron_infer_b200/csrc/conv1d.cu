// Mamba-2 depthwise causal conv1d (kernel 4) + bias + SiLU over the xBC projection, fused with the split of
// its output into the x | B | C tensors the scan consumes.
//
// The reference runs the convolution into one [M, conv_dim] tensor (ops/mamba2/causal_conv1d.cuh:369-389) and then
// copies that tensor out again in three strided cudaMemcpy2DAsync calls (model/mamba_block.cuh:199-207): every
// output byte crosses HBM three times (write, read, write).  Here the kernel stores each 16-byte vector
// straight into the segment it belongs to, so the traffic is one read of xBC and one write of x|B|C.
//
// Mapping: channels are contiguous within a row, so a thread owns one 16-byte vector of 8 channels and walks
// TIME_CHUNK consecutive time steps with the previous three inputs kept in registers (each input row is read
// once, plus three halo rows per chunk that the neighbouring chunk has just pulled into L2).  A warp covers
// 512 contiguous bytes of a row; loads are issued UNROLL steps ahead of their use.
#include "nmt_common.cuh"

namespace nmt {

constexpr int kConvTaps = 4;

// silu through the SFU (same form as the gated norm): x * 1 / (1 + 2^(-x log2 e)).
__device__ __forceinline__ float2 silu2_fast(const float2& v) {
    const float2 t = __fmul2_rn(v, make_float2(-1.4426950408889634f, -1.4426950408889634f));
    float2 e, rcp;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
    const float2 d = __fadd2_rn(e, make_float2(1.0f, 1.0f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp.x) : "f"(d.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp.y) : "f"(d.y));
    return __fmul2_rn(v, rcp);
}

// Scalar form: the conv accumulators come out of f32x2 FMAs, but feeding their halves to the SFU one by one and
// packing the two results straight into a bf16 pair avoids shuffling values between register pairs and
// single registers around every SFU instruction.
__device__ __forceinline__ float silu_fast(float v) {
    float e, rcp;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(v * -1.4426950408889634f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rcp) : "f"(1.0f + e));
    return v * rcp;
}
// (One reciprocal for a pair - 1/a = b / (ab), 1/b = a / (ab), three SFU instructions and three multiplies for four
// SFU instructions, with a guard where the product could overflow - was measured 25 % SLOWER at 65,536 tokens:
// the kernel is bound by the dependent-instruction chain per loaded vector at 64 registers, not by the SFU pipe.)

struct ConvSplit {          // conv_dim = n0 + n1 + n2 channels; segment i is a contiguous [M, n_i] tensor
    uint4* out[3];
    int nv[3];              // vectors (8 channels) per row of each segment
};

// A thread's slice of a row: NP channel pairs = 2*NP channels = 4*NP bytes (NP = 4: one 16-byte vector,
// NP = 2: one 8-byte vector, which halves the registers a thread needs and doubles the resident warps).
template <int NP> struct ConvVec;
template <> struct ConvVec<4> {
    using T = uint4;
    static __device__ __forceinline__ T ld(const T* p) { return ld_stream(p); }
    static __device__ __forceinline__ void st(T* p, const float2 (&o)[4]) { st_stream(p, pack8x2(o)); }
    static __device__ __forceinline__ void unpack(const T& v, float2 (&f)[4]) { unpack8x2(v, f); }
    static __device__ __forceinline__ T zero() { return make_uint4(0, 0, 0, 0); }
};
template <> struct ConvVec<2> {
    using T = uint2;
    static __device__ __forceinline__ T ld(const T* p) {
        T v;
        asm volatile("ld.global.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
        return v;
    }
    static __device__ __forceinline__ void st(T* p, const float2 (&o)[2]) {
        asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(pack2(o[0])), "r"(pack2(o[1])) : "memory");
    }
    static __device__ __forceinline__ void unpack(const T& v, float2 (&f)[2]) { f[0] = unpack2(v.x); f[1] = unpack2(v.y); }
    static __device__ __forceinline__ T zero() { return make_uint2(0, 0); }
};

template <int TIME_CHUNK, int UNROLL, int NP>
__global__ void __launch_bounds__(128, NP == 2 ? 8 : 4)     // 64 registers for the default (8-byte) form: 8 CTAs per SM instead of 7, +5 %
conv1d_silu_split_kernel(const void* __restrict__ xv, const float* __restrict__ w, const float* __restrict__ bias,
                         ConvSplit dst, float* state_out, int cv_total, int S, int batch) {
    using V = ConvVec<NP>;
    using VT = typename V::T;
    constexpr int CH = 2 * NP;                                     // channels per thread
    const VT* x = static_cast<const VT*>(xv);
    pdl_wait();
    const int cv = blockIdx.x * blockDim.x + threadIdx.x;          // which CH-channel vector of the row
    const int chunk = blockIdx.y;
    const int b = blockIdx.z;
    if (cv < cv_total) {
        const int t0 = chunk * TIME_CHUNK;
        const int t1 = min(t0 + TIME_CHUNK, S);
        const VT* xb = x + (size_t)b * S * cv_total + cv;

        // taps: w[ch][0..3] are contiguous, so one float4 per channel; regroup as (lo, hi) channel pairs per tap
        float2 wt[kConvTaps][NP], bs[NP];
#pragma unroll
        for (int p = 0; p < NP; ++p) {
            const float4 a = ld_weight4(w + ((size_t)cv * CH + 2 * p) * kConvTaps);
            const float4 c = ld_weight4(w + ((size_t)cv * CH + 2 * p + 1) * kConvTaps);
            wt[0][p] = make_float2(a.x, c.x); wt[1][p] = make_float2(a.y, c.y);
            wt[2][p] = make_float2(a.z, c.z); wt[3][p] = make_float2(a.w, c.w);
            bs[p] = make_float2(__ldg(bias + cv * CH + 2 * p), __ldg(bias + cv * CH + 2 * p + 1));
        }
        // which output segment this vector lands in (segment widths are in units of 8 channels)
        constexpr int PER8 = 8 / CH;                                // thread-vectors per 8 channels
        int seg = 0, col = cv;
        if (col >= dst.nv[0] * PER8) { col -= dst.nv[0] * PER8; seg = 1; if (col >= dst.nv[1] * PER8) { col -= dst.nv[1] * PER8; seg = 2; } }
        VT* outp = reinterpret_cast<VT*>(dst.out[seg]);
        const int onv = dst.nv[seg] * PER8;

        // sliding window: h[j] = x[t0 - 3 + j] (zero before the start of the sequence)
        float2 h[kConvTaps - 1][NP];
#pragma unroll
        for (int j = 0; j < kConvTaps - 1; ++j) {
            const int ti = t0 - (kConvTaps - 1) + j;
            const VT v = ti >= 0 ? V::ld(xb + (size_t)ti * cv_total) : V::zero();
            V::unpack(v, h[j]);
        }
        // One output step: bias, then taps oldest to newest, the reference's order (causal_conv1d.cuh:73-76).
        auto step = [&](const float2 (&a)[NP], const float2 (&b2)[NP], const float2 (&c)[NP], const float2 (&d)[NP], int t) {
            float2 o[NP];
#pragma unroll
            for (int p = 0; p < NP; ++p) {
                float2 acc = __ffma2_rn(wt[0][p], a[p], bs[p]);
                acc = __ffma2_rn(wt[1][p], b2[p], acc);
                acc = __ffma2_rn(wt[2][p], c[p], acc);
                acc = __ffma2_rn(wt[3][p], d[p], acc);
                o[p] = make_float2(silu_fast(acc.x), silu_fast(acc.y));
            }
            V::st(outp + ((size_t)b * S + t) * onv + col, o);
        };
        int tb = t0;
        // Full groups of UNROLL steps: all loads first, then a straight-line window v[0..UNROLL+2] with static
        // indices (no per-step predicate, so the window never has to be shuffled between registers).
        // (Issuing the next group's loads ahead of this group's arithmetic was tried: the extra registers cost
        // more occupancy than the overlap gained.  So was a per-thread cp.async ring of 16 / 32 time steps in
        // shared memory, which keeps 4x the bytes in flight at no register cost: bit-identical and 13-25 % slower,
        // so the bytes in flight are not what limits this kernel.)
        for (; tb + UNROLL <= t1; tb += UNROLL) {
            VT in[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) in[u] = V::ld(xb + (size_t)(tb + u) * cv_total);
            float2 v[UNROLL + 3][NP];
#pragma unroll
            for (int j = 0; j < 3; ++j)
#pragma unroll
                for (int p = 0; p < NP; ++p) v[j][p] = h[j][p];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                V::unpack(in[u], v[u + 3]);
                step(v[u], v[u + 1], v[u + 2], v[u + 3], tb + u);
            }
#pragma unroll
            for (int j = 0; j < 3; ++j)
#pragma unroll
                for (int p = 0; p < NP; ++p) h[j][p] = v[UNROLL + j][p];
        }
        // Ragged tail (S not a multiple of the chunk): one step at a time.
        for (; tb < t1; ++tb) {
            float2 cur[NP];
            V::unpack(V::ld(xb + (size_t)tb * cv_total), cur);
            step(h[0], h[1], h[2], cur, tb);
#pragma unroll
            for (int p = 0; p < NP; ++p) { h[0][p] = h[1][p]; h[1][p] = h[2][p]; h[2][p] = cur[p]; }
        }
        // the last chunk leaves the final three raw inputs for the decode step, [batch, conv_dim, 3] fp32
        if (t1 == S && state_out) {
            float* s = state_out + ((size_t)b * cv_total * CH + (size_t)cv * CH) * (kConvTaps - 1);
#pragma unroll
            for (int p = 0; p < NP; ++p) {
#pragma unroll
                for (int j = 0; j < kConvTaps - 1; ++j) {
                    s[(2 * p) * (kConvTaps - 1) + j] = h[j][p].x;
                    s[(2 * p + 1) * (kConvTaps - 1) + j] = h[j][p].y;
                }
            }
        }
    }
    pdl_trigger();
}

// Single-token form: one new xBC row per sequence, the three previous inputs come from (and the window goes back
// to) the fp32 state [batch, conv_dim, 3] that the prefill kernel left behind.  A thread owns 4 channels: 8 bytes of
// x, 48 contiguous bytes of state (three float4), 8 bytes of output stored straight into its x | B | C segment.
__global__ void __launch_bounds__(128)
conv1d_silu_decode_split_kernel(const uint2* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                ConvSplit dst, float* state, int cv_total, int batch) {
    pdl_wait();
    const int cv = blockIdx.x * blockDim.x + threadIdx.x;          // which 4-channel vector
    const int b = blockIdx.y;
    if (cv < cv_total) {
        const uint2 xv = x[(size_t)b * cv_total + cv];
        const float xin[4] = {bf16_lo(xv.x), bf16_hi(xv.x), bf16_lo(xv.y), bf16_hi(xv.y)};
        float4* sp = reinterpret_cast<float4*>(state + ((size_t)b * cv_total + cv) * 4 * (kConvTaps - 1));
        const float4 s0 = sp[0], s1 = sp[1], s2 = sp[2];
        const float st[12] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w, s2.x, s2.y, s2.z, s2.w};   // [channel][3]
        float o[4], ns[12];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const float4 wt = ld_weight4(w + ((size_t)cv * 4 + c) * kConvTaps);
            float acc = __ldg(bias + cv * 4 + c);                   // bias, then taps oldest to newest (causal_conv1d.cuh:415-418)
            acc = fmaf(wt.x, st[3 * c], acc);
            acc = fmaf(wt.y, st[3 * c + 1], acc);
            acc = fmaf(wt.z, st[3 * c + 2], acc);
            acc = fmaf(wt.w, xin[c], acc);
            o[c] = silu_fast(acc);
            ns[3 * c] = st[3 * c + 1];
            ns[3 * c + 1] = st[3 * c + 2];
            ns[3 * c + 2] = xin[c];
        }
        sp[0] = make_float4(ns[0], ns[1], ns[2], ns[3]);
        sp[1] = make_float4(ns[4], ns[5], ns[6], ns[7]);
        sp[2] = make_float4(ns[8], ns[9], ns[10], ns[11]);
        int seg = 0, col = cv;                                      // segment widths are in units of 8 channels = 2 vectors
        if (col >= dst.nv[0] * 2) { col -= dst.nv[0] * 2; seg = 1; if (col >= dst.nv[1] * 2) { col -= dst.nv[1] * 2; seg = 2; } }
        uint2* outp = reinterpret_cast<uint2*>(seg == 0 ? dst.out[0] : seg == 1 ? dst.out[1] : dst.out[2]);
        const int onv = (seg == 0 ? dst.nv[0] : seg == 1 ? dst.nv[1] : dst.nv[2]) * 2;
        outp[(size_t)b * onv + col] = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    }
    pdl_trigger();
}

// fp32 twin (parity with the golden emitter's stage tensors): one thread per (channel, chunk), scalar.
__global__ void __launch_bounds__(128)
conv1d_silu_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       float* y, float* state_out, int conv_dim, int S, int batch, int time_chunk) {
    pdl_wait();
    const int ch = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.z;
    if (ch < conv_dim) {
        const int t0 = blockIdx.y * time_chunk, t1 = min(t0 + time_chunk, S);
        const float* xb = x + (size_t)b * S * conv_dim + ch;
        float* yb = y + (size_t)b * S * conv_dim + ch;
        float wt[kConvTaps], h[kConvTaps - 1];
        for (int k = 0; k < kConvTaps; ++k) wt[k] = w[ch * kConvTaps + k];
        for (int j = 0; j < kConvTaps - 1; ++j) {
            const int ti = t0 - (kConvTaps - 1) + j;
            h[j] = ti >= 0 ? xb[(size_t)ti * conv_dim] : 0.f;
        }
        for (int t = t0; t < t1; ++t) {
            const float cur = xb[(size_t)t * conv_dim];
            float acc = bias[ch];
            acc = fmaf(wt[0], h[0], acc); acc = fmaf(wt[1], h[1], acc); acc = fmaf(wt[2], h[2], acc); acc = fmaf(wt[3], cur, acc);
            yb[(size_t)t * conv_dim] = acc / (1.f + expf(-acc));
            h[0] = h[1]; h[1] = h[2]; h[2] = cur;
        }
        if (t1 == S && state_out)
            for (int j = 0; j < kConvTaps - 1; ++j) state_out[((size_t)b * conv_dim + ch) * (kConvTaps - 1) + j] = h[j];
    }
    pdl_trigger();
}

}  // namespace nmt

extern "C" {

int nmt_causal_conv1d_silu_split_bf16(const void* xbc, const float* w, const float* bias, void* out0, void* out1,
                                      void* out2, int64_t n0, int64_t n1, int64_t n2, float* state_out,
                                      int64_t S, int64_t batch, void* stream) {
    using namespace nmt;
    if (S < 0 || batch < 0 || n0 <= 0 || n1 < 0 || n2 < 0 || (n0 % 8) || (n1 % 8) || (n2 % 8)) return NMT_ERR_SHAPE;
    if (S == 0 || batch == 0) return NMT_OK;
    if (!xbc || !w || !bias || !out0 || (n1 > 0 && !out1) || (n2 > 0 && !out2)) return NMT_ERR_NULL;
    if (!aligned16(xbc) || !aligned16(w) || !aligned4(bias) || !aligned16(out0) || (n1 > 0 && !aligned16(out1)) ||
        (n2 > 0 && !aligned16(out2)) || (state_out && !aligned4(state_out)))
        return NMT_ERR_ALIGN;
    if (batch > 65535 || S > (int64_t)65535 * 32) return NMT_ERR_UNSUPPORTED;
    ConvSplit dst;
    dst.out[0] = static_cast<uint4*>(out0); dst.out[1] = static_cast<uint4*>(out1); dst.out[2] = static_cast<uint4*>(out2);
    dst.nv[0] = static_cast<int>(n0 / 8); dst.nv[1] = static_cast<int>(n1 / 8); dst.nv[2] = static_cast<int>(n2 / 8);
    const int np = tune("conv.pairs", 2) >= 4 ? 4 : 2;            // channel pairs per thread
    const int cv_total = (dst.nv[0] + dst.nv[1] + dst.nv[2]) * (4 / np);
    const int tc = tune("conv.chunk", 64);
    const int time_chunk = tc >= 64 ? 64 : tc >= 32 ? 32 : tc >= 16 ? 16 : tc >= 8 ? 8 : 4;
    const int unroll = (tune("conv.unroll", 8) >= 8 && time_chunk >= 8) ? 8 : 4;
    const dim3 grid((cv_total + 127) / 128, static_cast<unsigned>((S + time_chunk - 1) / time_chunk), static_cast<unsigned>(batch));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(128);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
#define NMT_CONV_CASE(TC, UN)                                                                                      \
    do {                                                                                                           \
        if (np == 4) cudaLaunchKernelEx(&cfg, conv1d_silu_split_kernel<TC, UN, 4>, xbc, w, bias, dst, state_out,   \
                                        cv_total, static_cast<int>(S), static_cast<int>(batch));                   \
        else cudaLaunchKernelEx(&cfg, conv1d_silu_split_kernel<TC, UN, 2>, xbc, w, bias, dst, state_out,           \
                                cv_total, static_cast<int>(S), static_cast<int>(batch));                           \
    } while (0)
    if (time_chunk == 64 && unroll == 8) NMT_CONV_CASE(64, 8);
    else if (time_chunk == 64) NMT_CONV_CASE(64, 4);
    else if (time_chunk == 32 && unroll == 8) NMT_CONV_CASE(32, 8);
    else if (time_chunk == 32) NMT_CONV_CASE(32, 4);
    else if (time_chunk == 16 && unroll == 8) NMT_CONV_CASE(16, 8);
    else if (time_chunk == 16) NMT_CONV_CASE(16, 4);
    else if (time_chunk == 8 && unroll == 8) NMT_CONV_CASE(8, 8);
    else if (time_chunk == 8) NMT_CONV_CASE(8, 4);
    else NMT_CONV_CASE(4, 4);
#undef NMT_CONV_CASE
    return finish_launch(1);
}

int nmt_causal_conv1d_silu_decode_split_bf16(const void* xbc, const float* w, const float* bias, void* out0, void* out1,
                                             void* out2, int64_t n0, int64_t n1, int64_t n2, float* state, int64_t batch,
                                             void* stream) {
    using namespace nmt;
    if (batch < 0 || n0 <= 0 || n1 < 0 || n2 < 0 || (n0 % 8) || (n1 % 8) || (n2 % 8)) return NMT_ERR_SHAPE;
    if (batch == 0) return NMT_OK;
    if (!xbc || !w || !bias || !state || !out0 || (n1 > 0 && !out1) || (n2 > 0 && !out2)) return NMT_ERR_NULL;
    if (!aligned16(xbc) || !aligned16(w) || !aligned4(bias) || !aligned16(state) || !aligned16(out0) ||
        (n1 > 0 && !aligned16(out1)) || (n2 > 0 && !aligned16(out2)))
        return NMT_ERR_ALIGN;
    if (batch > 65535) return NMT_ERR_UNSUPPORTED;
    ConvSplit dst;
    dst.out[0] = static_cast<uint4*>(out0); dst.out[1] = static_cast<uint4*>(out1); dst.out[2] = static_cast<uint4*>(out2);
    dst.nv[0] = static_cast<int>(n0 / 8); dst.nv[1] = static_cast<int>(n1 / 8); dst.nv[2] = static_cast<int>(n2 / 8);
    const int cv_total = (dst.nv[0] + dst.nv[1] + dst.nv[2]) * 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((cv_total + 127) / 128, static_cast<unsigned>(batch));
    cfg.blockDim = dim3(128);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, conv1d_silu_decode_split_kernel, static_cast<const uint2*>(xbc), w, bias, dst, state, cv_total,
                       static_cast<int>(batch));
    return finish_launch(1);
}

int nmt_causal_conv1d_silu_f32(const float* x, const float* w, const float* bias, float* y, float* state_out,
                               int64_t conv_dim, int64_t S, int64_t batch, void* stream) {
    using namespace nmt;
    if (S < 0 || batch < 0 || conv_dim <= 0) return NMT_ERR_SHAPE;
    if (S == 0 || batch == 0) return NMT_OK;
    if (!x || !w || !bias || !y) return NMT_ERR_NULL;
    if (!aligned4(x) || !aligned4(w) || !aligned4(bias) || !aligned4(y) || (state_out && !aligned4(state_out))) return NMT_ERR_ALIGN;
    if (batch > 65535) return NMT_ERR_UNSUPPORTED;
    const int time_chunk = 64;
    const dim3 grid(static_cast<unsigned>((conv_dim + 127) / 128), static_cast<unsigned>((S + time_chunk - 1) / time_chunk),
                    static_cast<unsigned>(batch));
    conv1d_silu_f32_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(x, w, bias, y, state_out, static_cast<int>(conv_dim),
                                                                               static_cast<int>(S), static_cast<int>(batch), time_chunk);
    return finish_launch(1);
}

}  // extern "C"
