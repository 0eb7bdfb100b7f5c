// Attention for ONE query token over the KV cache (the decode step of the attention block, model/attention_block.cuh:
// 249-253, 403-406; replaces ops/attention/sdpa_decode.cuh:56-256, sdpa_decode_bf16<128>).
//
//   for every query head h (kv head g = h / (H_Q / H_KV)):   p = softmax_s(q_h . K[g, s] / sqrt(128)),  s < S_cache
//                                                            O[h] = sum_s p_s V[g, s]
//   then K_new / V_new are written to position S_cache of the cache (the new token does not attend to itself: that is
//   what the reference computes, and what its blocks are tested against).
//
// Bytes: the cache, once (2 x H_KV x S x 256 bytes: 2 MB at 512 cached tokens).  The reference gives every (query head,
// 128-position split) to one warp that walks its positions one after the other, so the five query heads of a group
// read the same K and V rows five times and a split is a chain of 128 dependent softmax updates.  Here a CTA owns a
// (kv head, split of 32 to 64 positions): each of its four warps takes every fourth position, reads the K and V row
// once (8 bytes per lane, four positions ahead) and updates all query heads of the group from it - independent chains
// that overlap - and the warps' partial (max, sum, output) are merged in shared memory.  A second launch merges the
// splits per query head, writes the output and appends the new K / V row.  Scratch for the partials comes from the
// caller.  Measured at 40 / 8 heads in a graph over cold caches: 4.8 / 5.7 / 9.8 / 14.9 / 45 / 93 us at 64 / 512 / 2048 /
// 4096 / 16,384 / 32,768 cached tokens (the reference's two kernels: 35 / 112 / 143 / 149 / 285 / 537 us).
#include <cfloat>

#include "nmt_common.cuh"

namespace nmt {

constexpr int kSdpaWarps = 4;
constexpr int kHeadDim = 128;
constexpr int kDPL = kHeadDim / 32;                                // head-dim elements per lane

// 2^x on the SFU (x <= 0 here).  Maxima and scores are kept in units of log 2: the 1 / sqrt(128) scale carries log2(e).
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void unpack4(const uint2& v, float (&f)[4]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
}

template <int RATIO>                                               // query heads per kv head
__global__ void __launch_bounds__(kSdpaWarps * 32)
sdpa_decode_partial_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K, const __nv_bfloat16* __restrict__ V,
                           int S_cache, int total_S, int chunk, int nsplit, float scale_log2, float* __restrict__ m_part,
                           float* __restrict__ l_part, float* __restrict__ o_part) {
    __shared__ float s_m[kSdpaWarps][RATIO], s_l[kSdpaWarps][RATIO];
    __shared__ __align__(16) float s_o[kSdpaWarps][RATIO][kHeadDim];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kv = blockIdx.x, split = blockIdx.y;
    const int s_begin = split * chunk, s_end = min(S_cache, s_begin + chunk);
    pdl_wait();
    float q[RATIO][kDPL], o[RATIO][kDPL], m[RATIO], l[RATIO];
#pragma unroll
    for (int r = 0; r < RATIO; ++r) {
        unpack4(*reinterpret_cast<const uint2*>(Q + (size_t)(kv * RATIO + r) * kHeadDim + lane * kDPL), q[r]);
        m[r] = -FLT_MAX;
        l[r] = 0.f;
#pragma unroll
        for (int i = 0; i < kDPL; ++i) o[r][i] = 0.f;
    }
    const size_t base = (size_t)kv * total_S * kHeadDim + lane * kDPL;
    // A warp's positions are s_begin + warp + 4 j.  They are handled four at a time, and the next four positions' K and V
    // rows are requested before the current four are used: 8 to 16 rows (2 to 4 KB) per warp on their way at any time.
    constexpr int GROUP = 4;
    uint2 kb[GROUP], vb[GROUP];
    auto load_group = [&](int s0, uint2 (&kk)[GROUP], uint2 (&vv)[GROUP]) {
#pragma unroll
        for (int a = 0; a < GROUP; ++a) {
            const int sa = s0 + a * kSdpaWarps;
            if (sa < s_end) {
                kk[a] = *reinterpret_cast<const uint2*>(K + base + (size_t)sa * kHeadDim);
                vv[a] = *reinterpret_cast<const uint2*>(V + base + (size_t)sa * kHeadDim);
            } else {
                kk[a] = make_uint2(0, 0);
                vv[a] = make_uint2(0, 0);
            }
        }
    };
    load_group(s_begin + warp, kb, vb);
    for (int s0 = s_begin + warp; s0 < s_end; s0 += GROUP * kSdpaWarps) {
        uint2 kn[GROUP], vn[GROUP];
        load_group(s0 + GROUP * kSdpaWarps, kn, vn);
#pragma unroll
        for (int a = 0; a < GROUP; ++a) {
            if (s0 + a * kSdpaWarps >= s_end) break;               // warp-uniform
            float kf[kDPL], vf[kDPL];
            unpack4(kb[a], kf);
            unpack4(vb[a], vf);
            float dot[RATIO];
#pragma unroll
            for (int r = 0; r < RATIO; ++r) {
                dot[r] = 0.f;
#pragma unroll
                for (int i = 0; i < kDPL; ++i) dot[r] = fmaf(q[r][i], kf[i], dot[r]);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                for (int r = 0; r < RATIO; ++r) dot[r] += __shfl_xor_sync(0xffffffffu, dot[r], off);
            }
#pragma unroll
            for (int r = 0; r < RATIO; ++r) {
                // online softmax: of the two factors exp(m - m_new) and exp(score - m_new) one is always exactly 1
                const float score = dot[r] * scale_log2;
                const float e = exp2_fast(-fabsf(score - m[r]));
                const bool up = score > m[r];
                const float corr = up ? e : 1.f, p = up ? 1.f : e;
#pragma unroll
                for (int i = 0; i < kDPL; ++i) o[r][i] = fmaf(o[r][i], corr, p * vf[i]);
                l[r] = fmaf(l[r], corr, p);
                m[r] = fmaxf(m[r], score);
            }
        }
#pragma unroll
        for (int a = 0; a < GROUP; ++a) { kb[a] = kn[a]; vb[a] = vn[a]; }
    }
    // merge the warps: standard rescaling to the common maximum, warps in order
#pragma unroll
    for (int r = 0; r < RATIO; ++r) {
        if (lane == 0) { s_m[warp][r] = m[r]; s_l[warp][r] = l[r]; }
        *reinterpret_cast<float4*>(&s_o[warp][r][lane * kDPL]) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
    }
    __syncthreads();
    const int d = threadIdx.x;                                     // kSdpaWarps * 32 == kHeadDim threads: one per output element
#pragma unroll
    for (int r = 0; r < RATIO; ++r) {
        float gm = -FLT_MAX;
#pragma unroll
        for (int w = 0; w < kSdpaWarps; ++w) gm = fmaxf(gm, s_m[w][r]);
        float gl = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kSdpaWarps; ++w) {
            const float sc = exp2_fast(s_m[w][r] - gm);
            gl = fmaf(sc, s_l[w][r], gl);
            acc = fmaf(sc, s_o[w][r][d], acc);
        }
        const size_t pidx = (size_t)(kv * RATIO + r) * nsplit + split;
        o_part[pidx * kHeadDim + d] = acc;
        if (d == 0) { m_part[pidx] = gm; l_part[pidx] = gl; }
    }
    pdl_trigger();
}

// One CTA per query head: merge the splits, normalise, append the new K / V row.  Thread (slice, d) merges every
// kCombineSlices-th split for output element d; the slices are merged in shared memory.
constexpr int kCombineSlices = 4;
__global__ void __launch_bounds__(kHeadDim * kCombineSlices)
sdpa_decode_combine_kernel(__nv_bfloat16* __restrict__ O, __nv_bfloat16* __restrict__ K, __nv_bfloat16* __restrict__ V,
                           const __nv_bfloat16* __restrict__ K_new, const __nv_bfloat16* __restrict__ V_new,
                           const float* __restrict__ m_part, const float* __restrict__ l_part, const float* __restrict__ o_part,
                           int ratio, int nsplit, int S_cache, int total_S) {
    __shared__ float s_m[kCombineSlices], s_l[kCombineSlices], s_acc[kCombineSlices][kHeadDim];
    const int head = blockIdx.x, d = threadIdx.x & (kHeadDim - 1), slice = threadIdx.x / kHeadDim;
    // the new row first: K_new / V_new come from launches before the partial kernel, the cache slot is nobody's input
    if (slice == 0 && head % ratio == 0) {
        const int kv = head / ratio;
        const size_t slot = ((size_t)kv * total_S + S_cache) * kHeadDim + d;
        K[slot] = K_new[(size_t)kv * kHeadDim + d];
        V[slot] = V_new[(size_t)kv * kHeadDim + d];
    }
    pdl_wait();
    float gm = -FLT_MAX;
    for (int sp = slice; sp < nsplit; sp += kCombineSlices) gm = fmaxf(gm, m_part[head * nsplit + sp]);
    float gl = 0.f, acc = 0.f;
    for (int sp = slice; sp < nsplit; sp += kCombineSlices) {
        const int pidx = head * nsplit + sp;
        const float w = exp2_fast(m_part[pidx] - gm);
        gl = fmaf(w, l_part[pidx], gl);
        acc = fmaf(w, o_part[(size_t)pidx * kHeadDim + d], acc);
    }
    if (d == 0) { s_m[slice] = gm; s_l[slice] = gl; }
    s_acc[slice][d] = acc;
    __syncthreads();
    if (slice == 0) {
        float tm = -FLT_MAX;
#pragma unroll
        for (int c = 0; c < kCombineSlices; ++c) tm = fmaxf(tm, s_m[c]);
        float tl = 0.f, ta = 0.f;
#pragma unroll
        for (int c = 0; c < kCombineSlices; ++c) {
            const float w = exp2_fast(s_m[c] - tm);                // an empty slice has l = acc = 0: its weight does not matter
            tl = fmaf(w, s_l[c], tl);
            ta = fmaf(w, s_acc[c][d], ta);
        }
        const float inv = tl > 0.f ? 1.f / tl : 0.f;
        O[(size_t)head * kHeadDim + d] = __float2bfloat16_rn(ta * inv);
    }
    pdl_trigger();
}

// Splits of 32 positions (8 per warp) up to 1024 cached tokens, of 64 beyond, at most 512 of them.
static int sdpa_splits(int64_t S_cache) {
    int64_t n = S_cache <= 1024 ? (S_cache + 31) / 32 : (S_cache + 63) / 64;
    return static_cast<int>(n < 1 ? 1 : n > 512 ? 512 : n);
}

}  // namespace nmt

extern "C" {

int64_t nmt_sdpa_decode_workspace_bytes(int64_t S_cache, int64_t num_heads) {
    if (S_cache < 0 || num_heads <= 0) return 0;
    return num_heads * nmt::sdpa_splits(S_cache) * (nmt::kHeadDim + 2) * static_cast<int64_t>(sizeof(float));
}

int nmt_sdpa_decode_bf16(const void* Q, void* K_cache, void* V_cache, void* O, const void* K_new, const void* V_new,
                         int64_t S_cache, int64_t total_S, int64_t num_heads, int64_t num_kv_heads, int64_t head_dim,
                         void* workspace, void* stream) {
    using namespace nmt;
    if (num_kv_heads <= 0) num_kv_heads = num_heads;
    if (num_heads <= 0 || S_cache < 0 || total_S <= S_cache || (num_heads % num_kv_heads) != 0) return NMT_ERR_SHAPE;
    const int64_t ratio = num_heads / num_kv_heads;
    if (head_dim != kHeadDim || !(ratio == 1 || ratio == 2 || ratio == 4 || ratio == 5 || ratio == 8) || num_kv_heads > 0x7fffffff ||
        total_S > 0x7fffffff)
        return NMT_ERR_UNSUPPORTED;
    if (!Q || !K_cache || !V_cache || !O || !K_new || !V_new || !workspace) return NMT_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(Q) & 7u) || (reinterpret_cast<uintptr_t>(K_cache) & 7u) || (reinterpret_cast<uintptr_t>(V_cache) & 7u) ||
        (reinterpret_cast<uintptr_t>(O) & 1u) || (reinterpret_cast<uintptr_t>(K_new) & 1u) || (reinterpret_cast<uintptr_t>(V_new) & 1u) ||
        !aligned16(workspace))
        return NMT_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nsplit = sdpa_splits(S_cache);
    const int chunk = static_cast<int>((S_cache + nsplit - 1) / nsplit);
    float* o_part = static_cast<float*>(workspace);                // [heads][nsplit][128], then the two [heads][nsplit] arrays
    float* m_part = o_part + num_heads * nsplit * kHeadDim;
    float* l_part = m_part + num_heads * nsplit;
    auto Qp = static_cast<const __nv_bfloat16*>(Q);
    auto Kp = static_cast<__nv_bfloat16*>(K_cache);
    auto Vp = static_cast<__nv_bfloat16*>(V_cache);
    const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(kHeadDim));     // log2(e) / sqrt(d)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(num_kv_heads), static_cast<unsigned>(nsplit));
    cfg.blockDim = dim3(kSdpaWarps * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
#define NMT_SDPA_CASE(R)                                                                                                  \
    cudaLaunchKernelEx(&cfg, sdpa_decode_partial_kernel<R>, Qp, static_cast<const __nv_bfloat16*>(Kp),                   \
                       static_cast<const __nv_bfloat16*>(Vp), static_cast<int>(S_cache), static_cast<int>(total_S), chunk, nsplit, \
                       scale_log2, m_part, l_part, o_part)
    switch (ratio) {
        case 1: NMT_SDPA_CASE(1); break;
        case 2: NMT_SDPA_CASE(2); break;
        case 4: NMT_SDPA_CASE(4); break;
        case 5: NMT_SDPA_CASE(5); break;
        default: NMT_SDPA_CASE(8); break;
    }
#undef NMT_SDPA_CASE
    launch_kernel(sdpa_decode_combine_kernel, static_cast<int>(num_heads), kHeadDim * kCombineSlices, 0, st, static_cast<__nv_bfloat16*>(O), Kp, Vp,
                  static_cast<const __nv_bfloat16*>(K_new), static_cast<const __nv_bfloat16*>(V_new),
                  static_cast<const float*>(m_part), static_cast<const float*>(l_part), static_cast<const float*>(o_part),
                  static_cast<int>(ratio), nsplit, static_cast<int>(S_cache), static_cast<int>(total_S));
    return finish_launch(2);
}

}  // extern "C"
