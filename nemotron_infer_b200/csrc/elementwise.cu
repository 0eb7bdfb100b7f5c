// relu^2 activation and residual add: pure streams (one read or two, one write).
//
// Register variant: a CTA takes a tile of blockDim * U 16-byte vectors; every
// thread issues its U loads (stride blockDim, so each warp request is 512
// contiguous bytes) before the first use, which keeps U * 16 B * threads in
// flight per CTA.  The arithmetic is packed bf16x2: a relu-clamped FMA then a
// bf16 multiply (x*x is exact in fp32, so the single bf16 rounding equals
// "square in fp32, round to nearest even"); add is one bf16x2 add (single
// rounding of the exact sum).
#include "nmt_common.cuh"

namespace nmt {

enum { kOpRelu2 = 0, kOpAdd = 1 };

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hadd2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
template <int OP>
__device__ __forceinline__ uint4 apply_op(const uint4& a, const uint4& b) {
    uint4 o;
    if (OP == kOpRelu2) {
        o.x = relu2_bf16x2(a.x); o.y = relu2_bf16x2(a.y); o.z = relu2_bf16x2(a.z); o.w = relu2_bf16x2(a.w);
    } else {
        o.x = add_bf16x2(a.x, b.x); o.y = add_bf16x2(a.y, b.y); o.z = add_bf16x2(a.z, b.z); o.w = add_bf16x2(a.w, b.w);
    }
    return o;
}

template <int OP, int U, int MAXB>
__global__ void __launch_bounds__(MAXB)
ew_stream_kernel(const uint4* a, const uint4* b, uint4* out, int64_t nv) {
    pdl_wait();
    const int64_t tile_vecs = (int64_t)blockDim.x * U;
#pragma unroll 1
    for (int64_t base = (int64_t)blockIdx.x * tile_vecs; base < nv; base += (int64_t)gridDim.x * tile_vecs) {
        uint4 va[U], vb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = base + (int64_t)u * blockDim.x + threadIdx.x;
            if (i < nv) {
                va[u] = ld_stream(a + i);
                if (OP == kOpAdd) vb[u] = ld_stream(b + i);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = base + (int64_t)u * blockDim.x + threadIdx.x;
            if (i < nv) st_stream(out + i, apply_op<OP>(va[u], vb[u]));
        }
    }
    pdl_trigger();
}

// fp32 twins (parity only).  relu2 follows torch: NaN in, NaN out.
template <int OP>
__global__ void __launch_bounds__(256)
ew_f32_kernel(const float* a, const float* b, float* out, int64_t n) {
    pdl_wait();
#pragma unroll 1
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float x = a[i];
        if (OP == kOpRelu2) out[i] = x > 0.f ? x * x : (x == x ? 0.f : x);
        else out[i] = x + b[i];
    }
    pdl_trigger();
}

template <int OP>
static int launch_ew_bf16(const void* a, const void* b, void* out, int64_t n, cudaStream_t st) {
    const int64_t nv = n / 8;
    int block = tune("ew.block", 512);
    const int unroll = tune("ew.unroll", 2);
    if (block > 1024) block = 1024;
    block = (block + 31) / 32 * 32;
    const int per_sm = tune("ew.ctas_per_sm", 0);
    auto A = static_cast<const uint4*>(a);
    auto B = static_cast<const uint4*>(b);
    auto O = static_cast<uint4*>(out);
#define NMT_EW_CASE(U)                                                                              \
    do {                                                                                            \
        const int grid = grid_for(nv, block * U, per_sm > 0 ? kSmCount * per_sm : 0x7fffffff);      \
        if (block <= 256) launch_kernel(ew_stream_kernel<OP, U, 256>, grid, block, 0, st, A, B, O, nv);        \
        else launch_kernel(ew_stream_kernel<OP, U, 1024>, grid, block, 0, st, A, B, O, nv);                    \
    } while (0)
    if (unroll >= 16) NMT_EW_CASE(16);
    else if (unroll >= 8) NMT_EW_CASE(8);
    else if (unroll >= 4) NMT_EW_CASE(4);
    else if (unroll >= 2) NMT_EW_CASE(2);
    else NMT_EW_CASE(1);
#undef NMT_EW_CASE
    return finish_launch(1);
}

static int check_ew(const void* a, const void* b, const void* out, int64_t n, bool binary, bool bf16) {
    if (n < 0 || (bf16 && (n % 8) != 0)) return NMT_ERR_SHAPE;
    if (n == 0) return NMT_OK;
    if (!a || !out || (binary && !b)) return NMT_ERR_NULL;
    if (bf16) {
        if (!aligned16(a) || !aligned16(out) || (binary && !aligned16(b))) return NMT_ERR_ALIGN;
    } else {
        if (!aligned4(a) || !aligned4(out) || (binary && !aligned4(b))) return NMT_ERR_ALIGN;
    }
    return NMT_OK;
}

}  // namespace nmt

extern "C" {

int nmt_relu2_bf16(const void* u, void* out, int64_t n, void* stream) {
    int s = nmt::check_ew(u, nullptr, out, n, false, true);
    if (s != NMT_OK || n == 0) return s;
    return nmt::launch_ew_bf16<nmt::kOpRelu2>(u, nullptr, out, n, static_cast<cudaStream_t>(stream));
}

int nmt_add_bf16(const void* a, const void* b, void* out, int64_t n, void* stream) {
    int s = nmt::check_ew(a, b, out, n, true, true);
    if (s != NMT_OK || n == 0) return s;
    return nmt::launch_ew_bf16<nmt::kOpAdd>(a, b, out, n, static_cast<cudaStream_t>(stream));
}

int nmt_relu2_f32(const float* u, float* out, int64_t n, void* stream) {
    int s = nmt::check_ew(u, nullptr, out, n, false, false);
    if (s != NMT_OK || n == 0) return s;
    const int grid = nmt::grid_for(n, 256 * 4, nmt::kSmCount * 16);
    nmt::launch_kernel(nmt::ew_f32_kernel<nmt::kOpRelu2>, grid, 256, 0, static_cast<cudaStream_t>(stream), u, nullptr, out, n);
    return nmt::finish_launch(1);
}

int nmt_add_f32(const float* a, const float* b, float* out, int64_t n, void* stream) {
    int s = nmt::check_ew(a, b, out, n, true, false);
    if (s != NMT_OK || n == 0) return s;
    const int grid = nmt::grid_for(n, 256 * 4, nmt::kSmCount * 16);
    nmt::launch_kernel(nmt::ew_f32_kernel<nmt::kOpAdd>, grid, 256, 0, static_cast<cudaStream_t>(stream), a, b, out, n);
    return nmt::finish_launch(1);
}

}  // extern "C"
