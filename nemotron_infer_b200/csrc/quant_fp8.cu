// Per-tensor dynamic FP8 (e4m3) quantisation of activations, alone and fused with the op that produces them.
//
// The reference quantises every FP8 GEMM input in two extra passes over a bf16 tensor it has just written
// (ops/gemm.cuh:257-307: an amax reduction on at most 1024 CTAs, then the quantiser), after the RMSNorm or
// relu^2 kernel that produced that tensor.  Here:
//   * nmt_quantize_fp8            same two steps, same arithmetic, full-width vectorised grids;
//   * nmt_[add_]rmsnorm_quant_fp8 pass 1 reads x (and r), writes the residual stream, and keeps only the
//                                 row's rstd (4 bytes) and the running |max| of the normed row; pass 2 reads
//                                 the residual stream back and writes e4m3 directly.  The bf16 normed tensor
//                                 is never written or re-read: 28.2 KB per 3136-wide token instead of 47 KB;
//   * nmt_relu2_quant_fp8         pass 1 only reads u (max of the positive part), pass 2 reads u again and
//                                 writes e4m3: 5 bytes per element instead of 9, the bf16 activation tensor
//                                 never exists.
// Rounding to bf16 and to e4m3 is monotone, so the maximum of the rounded values is the rounded maximum: the
// passes track the maximum of unrounded fp32 magnitudes and round once, and every result equals what the
// unfused sequence "op -> bf16 tensor -> amax -> quantise" produces from the same op output.
#include <cuda_fp8.h>

#include "nmt_common.cuh"

namespace nmt {

constexpr float kE4M3Max = 448.f;

// scale = amax / 448 (1/448 when the tensor is all zero), as ops/gemm.cuh:279-283.
__device__ __forceinline__ float scale_from_amax(float amax) {
    float s = amax / kE4M3Max;
    if (s < 1e-10f) s = 1.f / kE4M3Max;
    return s;
}
// Two values -> two e4m3 bytes.  The reference clamps to [-448, 448] with fminf / fmaxf and then converts
// (ops/gemm.cuh:286-288); the conversion used here saturates by itself, so only the upper clamp is kept: it is
// what turns a NaN into +448 (fminf returns its non-NaN operand), and every value the lower clamp would have
// changed (below -448, including -inf) is saturated to -448 by the conversion.  The product runs as one f32x2
// multiply.
__device__ __forceinline__ uint32_t quant2(const float2& v, const float2& inv2) {
    const float2 q = __fmul2_rn(v, inv2);
    uint32_t r;
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }"
        : "=r"(r) : "f"(fminf(kE4M3Max, q.y)), "f"(fminf(kE4M3Max, q.x)));
    return r;
}
// Eight bf16 values (one 16-byte vector) -> eight e4m3 bytes.
__device__ __forceinline__ uint2 quant8(const uint4& v, float inv) {
    const float2 inv2 = make_float2(inv, inv);
    uint2 o;
    o.x = quant2(unpack2(v.x), inv2) | (quant2(unpack2(v.y), inv2) << 16);
    o.y = quant2(unpack2(v.z), inv2) | (quant2(unpack2(v.w), inv2) << 16);
    return o;
}
__device__ __forceinline__ void st_stream8(uint2* p, const uint2& v) {
    asm volatile("st.global.L1::no_allocate.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}
enum { kXfIdentity = 0, kXfRelu2 = 1 };

// ---------------------------------------------------------------------------------------------
// Flat tensors: amax pass and quantising pass, optionally through relu^2.
// ---------------------------------------------------------------------------------------------
template <int XF, int U>
__global__ void __launch_bounds__(512)
amax_kernel(const uint4* x, unsigned int* amax_word, int64_t nv) {
    pdl_wait();
    float m = 0.f;
    const int64_t tile = (int64_t)blockDim.x * U;
#pragma unroll 1
    for (int64_t base = (int64_t)blockIdx.x * tile; base < nv; base += (int64_t)gridDim.x * tile) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = base + (int64_t)u * blockDim.x + threadIdx.x;
            v[u] = i < nv ? ld_stream(x + i) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float f[8];
            unpack8(v[u], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) m = fmaxf(m, XF == kXfRelu2 ? f[k] : fabsf(f[k]));   // relu: positive part only
        }
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0 && m > 0.f) publish_max(amax_word, m);
    pdl_trigger();
}

template <int XF, int U>
__global__ void __launch_bounds__(512)
quant_kernel(const uint4* x, uint2* out, const unsigned int* amax_word, float* scale_out, int64_t nv) {
    pdl_wait();
    float amax = __uint_as_float(*amax_word);
    if (XF == kXfRelu2) amax = bf16_round(amax * amax);      // the word holds max(u, 0); the tensor is its square
    const float s = scale_from_amax(amax);
    const float inv = 1.f / s;
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = s;
    const int64_t tile = (int64_t)blockDim.x * U;
#pragma unroll 1
    for (int64_t base = (int64_t)blockIdx.x * tile; base < nv; base += (int64_t)gridDim.x * tile) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = base + (int64_t)u * blockDim.x + threadIdx.x;
            if (i < nv) v[u] = ld_stream(x + i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = base + (int64_t)u * blockDim.x + threadIdx.x;
            if (i < nv) {
                uint4 a = v[u];
                if (XF == kXfRelu2) {           // act = bf16(relu(u)^2), exactly the relu^2 kernel's output
                    a.x = relu2_bf16x2(a.x); a.y = relu2_bf16x2(a.y); a.z = relu2_bf16x2(a.z); a.w = relu2_bf16x2(a.w);
                }
                st_stream8(out + i, quant8(a, inv));
            }
        }
    }
    pdl_trigger();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm (optionally with the residual add) fused with the quantisation statistics, then the quantiser.
// ---------------------------------------------------------------------------------------------
template <int SLOTS, bool FUSE_ADD>
__global__ void __launch_bounds__(512)
norm_stats_kernel(const uint4* x, const uint4* r, const float* __restrict__ w, uint4* out_res,
                  float* rstd_out, unsigned int* amax_word, int64_t rows, int nv, float inv_cols, float eps,
                  bool butterfly) {
    pdl_wait();
    __shared__ __align__(16) float s_part[2][16];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    int flip = 0;
    float m = 0.f;
#pragma unroll 1
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, flip ^= 1) {
        uint4 a[SLOTS], b[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int v = s * blockDim.x + threadIdx.x;
            if (v < nv) {
                a[s] = ld_stream(x + row * nv + v);
                if (FUSE_ADD) b[s] = ld_stream(r + row * nv + v);
            } else {
                a[s] = make_uint4(0, 0, 0, 0);
                if (FUSE_ADD) b[s] = make_uint4(0, 0, 0, 0);
            }
        }
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            if (FUSE_ADD) {
                a[s] = add_bf16x8_rn(a[s], b[s]);
                const int v = s * blockDim.x + threadIdx.x;
                if (v < nv) st_stream(out_res + row * nv + v, a[s]);
            }
            float2 p[4];
            unpack8x2(a[s], p);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc = __ffma2_rn(p[k], p[k], acc);
        }
        const float ss = warp_sum(acc.x + acc.y);
        if (lane == 0) s_part[flip][wid] = ss;
        __syncthreads();
        // The warps' partial sums are added in the order of the kernel nmt_rmsnorm_bf16 runs at this width, so that
        // rstd (and with it every output byte) equals the unfused norm's: sequentially for the register kernel, as a
        // butterfly for the shared-memory-staged kernel that takes plain norms of 20,488 - 32,768 columns.
        float total = 0.f;
        if (butterfly) total = warp_sum(lane < nwarps ? s_part[flip][lane] : 0.f);
        else for (int i = 0; i < nwarps; ++i) total += s_part[flip][i];
        const float rstd = rsqrtf(total * inv_cols + eps);
        if (threadIdx.x == 0) rstd_out[row] = rstd;
        const float2 rs = make_float2(rstd, rstd);
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int v = s * blockDim.x + threadIdx.x;
            if (v < nv) {
                float2 p[4];
                unpack8x2(a[s], p);
                const float4 w0 = ld_weight4(w + v * 8), w1 = ld_weight4(w + v * 8 + 4);
                const float2 o0 = __fmul2_rn(__fmul2_rn(p[0], rs), make_float2(w0.x, w0.y));
                const float2 o1 = __fmul2_rn(__fmul2_rn(p[1], rs), make_float2(w0.z, w0.w));
                const float2 o2 = __fmul2_rn(__fmul2_rn(p[2], rs), make_float2(w1.x, w1.y));
                const float2 o3 = __fmul2_rn(__fmul2_rn(p[3], rs), make_float2(w1.z, w1.w));
                m = fmaxf(m, fmaxf(fmaxf(fmaxf(fabsf(o0.x), fabsf(o0.y)), fmaxf(fabsf(o1.x), fabsf(o1.y))),
                                   fmaxf(fmaxf(fabsf(o2.x), fabsf(o2.y)), fmaxf(fabsf(o3.x), fabsf(o3.y)))));
            }
        }
    }
    m = warp_max(m);
    if (lane == 0 && m > 0.f) publish_max(amax_word, bf16_round(m));   // the tensor that is quantised is bf16
    pdl_trigger();
}

template <int SLOTS, int ROWS>
__global__ void __launch_bounds__(512)
norm_quant_kernel(const uint4* h, const float* __restrict__ w, const float* __restrict__ rstd_in,
                  const unsigned int* amax_word, uint2* out, float* scale_out, int64_t rows, int nv) {
    pdl_wait();
    const float s = scale_from_amax(__uint_as_float(*amax_word));
    const float inv = 1.f / s;
    if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = s;
    // ROWS rows per CTA pass: this kernel moves only 1.5 bytes per element, so a CTA needs several rows'
    // worth of loads in flight to be worth its launch.
#pragma unroll 1
    for (int64_t row0 = (int64_t)blockIdx.x * ROWS; row0 < rows; row0 += (int64_t)gridDim.x * ROWS) {
        uint4 a[ROWS][SLOTS];
        float rstd[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int64_t row = row0 + r;
            rstd[r] = row < rows ? __ldg(rstd_in + row) : 0.f;
#pragma unroll
            for (int q = 0; q < SLOTS; ++q) {
                const int v = q * blockDim.x + threadIdx.x;
                if (row < rows && v < nv) a[r][q] = ld_stream(h + row * nv + v);
            }
        }
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int v = q * blockDim.x + threadIdx.x;
            if (v < nv) {
                const float4 w0 = ld_weight4(w + v * 8), w1 = ld_weight4(w + v * 8 + 4);
#pragma unroll
                for (int r = 0; r < ROWS; ++r) {
                    const int64_t row = row0 + r;
                    if (row < rows) {
                        float2 p[4];
                        unpack8x2(a[r][q], p);
                        const uint4 normed = scale8(p, rstd[r], w0, w1);      // bf16, as the norm kernel writes it
                        st_stream8(out + row * nv + v, quant8(normed, inv));
                    }
                }
            }
        }
    }
    pdl_trigger();
}

static int ew_grid(int64_t nv, int block, int unroll) {
    return grid_for(nv, block * unroll, kSmCount * 32);
}

template <int XF>
static int launch_quant_flat(const void* x, void* out, float* scale_out, unsigned int* amax_word, int64_t n,
                             cudaStream_t st) {
    if (n < 0 || (n % 8) != 0) return NMT_ERR_SHAPE;
    if (n == 0) return NMT_OK;
    if (!x || !out || !amax_word) return NMT_ERR_NULL;
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(out) & 7u) || !aligned4(amax_word) || (scale_out && !aligned4(scale_out)))
        return NMT_ERR_ALIGN;
    const int64_t nv = n / 8;
    if (cudaMemsetAsync(amax_word, 0, sizeof(unsigned int), st) != cudaSuccess) return finish_launch(0);
    constexpr int U = 4, B = 256;
    launch_kernel(amax_kernel<XF, U>, ew_grid(nv, B, U), B, 0, st, static_cast<const uint4*>(x), amax_word, nv);
    launch_kernel(quant_kernel<XF, U>, ew_grid(nv, B, U), B, 0, st, static_cast<const uint4*>(x), static_cast<uint2*>(out),
                  static_cast<const unsigned int*>(amax_word), scale_out, nv);
    return finish_launch(2);
}


template <bool FUSE_ADD>
static int launch_norm_quant(const void* x, const void* r, const float* w, void* out_res, void* out_fp8,
                             float* scale_out, void* workspace, int64_t rows, int64_t cols, float eps, cudaStream_t st) {
    if (rows < 0 || cols <= 0 || (cols % 8) != 0) return NMT_ERR_SHAPE;
    if (rows == 0) return NMT_OK;
    if (!x || !w || !out_fp8 || !workspace || (FUSE_ADD && (!r || !out_res))) return NMT_ERR_NULL;
    if (!aligned16(x) || !aligned16(w) || (reinterpret_cast<uintptr_t>(out_fp8) & 7u) || !aligned16(workspace) ||
        (FUSE_ADD && (!aligned16(r) || !aligned16(out_res))) || (scale_out && !aligned4(scale_out)))
        return NMT_ERR_ALIGN;
    const int64_t nv = cols / 8;
    if (nv > 8 * 512) return NMT_ERR_UNSUPPORTED;
    unsigned int* amax_word = static_cast<unsigned int*>(workspace);
    float* rstd = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    if (cudaMemsetAsync(amax_word, 0, sizeof(unsigned int), st) != cudaSuccess) return finish_launch(0);
    const int block = default_norm_block(nv, FUSE_ADD);
    const int slots = static_cast<int>((nv + block - 1) / block);
    const int grid = grid_for(rows, 1, 0x7fffffff);
    const int qrows = tune("quant.rows_per_cta", 2);
    const bool butterfly = !FUSE_ADD && nv > 2560 && tune("norm.cluster", 0) == 0 && tune("norm.staged_single", 1) == 1;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    auto X = static_cast<const uint4*>(x);
    auto R = static_cast<const uint4*>(r);
    auto OR = static_cast<uint4*>(out_res);
    const uint4* H = FUSE_ADD ? static_cast<const uint4*>(out_res) : X;
    auto Q = static_cast<uint2*>(out_fp8);
#define NMT_NQ_CASE(S)                                                                                          \
    do {                                                                                                        \
        launch_kernel(norm_stats_kernel<S, FUSE_ADD>, grid, block, 0, st, X, R, w, OR, rstd, amax_word, rows,   \
                      (int)nv, inv_cols, eps, butterfly);                                                                \
        if (qrows >= 4) launch_kernel(norm_quant_kernel<S, 4>, grid_for(rows, 4, 0x7fffffff), block, 0, st, H, w, static_cast<const float*>(rstd), \
                      static_cast<const unsigned int*>(amax_word), Q, scale_out, rows, (int)nv);                \
        else if (qrows >= 2) launch_kernel(norm_quant_kernel<S, 2>, grid_for(rows, 2, 0x7fffffff), block, 0, st, H, w, static_cast<const float*>(rstd), \
                      static_cast<const unsigned int*>(amax_word), Q, scale_out, rows, (int)nv);                \
        else launch_kernel(norm_quant_kernel<S, 1>, grid_for(rows, 1, 0x7fffffff), block, 0, st, H, w, static_cast<const float*>(rstd), \
                      static_cast<const unsigned int*>(amax_word), Q, scale_out, rows, (int)nv);                \
    } while (0)
    if (slots <= 1) NMT_NQ_CASE(1);
    else if (slots <= 2) NMT_NQ_CASE(2);
    else if (slots <= 3) NMT_NQ_CASE(3);
    else if (slots <= 4) NMT_NQ_CASE(4);
    else if (slots <= 6) NMT_NQ_CASE(6);
    else NMT_NQ_CASE(8);
#undef NMT_NQ_CASE
    return finish_launch(2);
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for nmt_add_rmsnorm_quant_fp8_static.
//
// The fused norm + quantise pair needs a little device memory between its two kernels: one word for the
// running maximum and one float per row.  Some hosts have nowhere to get it from.  The reference's own
// engine is one: it forbids cudaMalloc / cudaFree anywhere inside the per-layer loop (cudaFree stalls the
// whole device, ops/gemm.cuh:322-323, binding.cu:58) and its bump allocator may have no slab left to carve from.  A thin
// ctypes / cgo style binding is another: it only ever sees the tensor addresses the engine hands it and owns
// no device allocator at all.  And a serving process that has given every free byte to its KV cache cannot
// count on a late cudaMalloc to succeed.  For those callers the scratch lives inside the library image:
// this array is part of the module, so it exists (on every GPU that loads the library, until the process
// exits) without anyone allocating it.
//
// kStaticMaxRows bounds it: 256 bytes of header plus 4 bytes per row = 262,400 bytes per GPU.
// ---------------------------------------------------------------------------------------------
constexpr int64_t kStaticMaxRows = NMT_STATIC_SCRATCH_MAX_ROWS;
static __device__ __align__(256) unsigned char g_fp8_static_scratch[256 + 4 * kStaticMaxRows];

// In host code the array's name is only a handle for the runtime, not an address a kernel could use; the
// device address has to be asked for, per device, with that device current.  It is looked up once per device
// and remembered.
static void* static_scratch_address(int* status) {
    static void* per_device[64] = {};
    static std::atomic<int> lock{0};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *status = finish_launch(0); if (*status == NMT_OK) *status = NMT_ERR_LAUNCH; return nullptr; }
    while (lock.exchange(1, std::memory_order_acquire)) {}
    void* p = per_device[dev];
    if (!p) {
        void* sym = nullptr;
        if (cudaGetSymbolAddress(&sym, g_fp8_static_scratch) == cudaSuccess && sym) per_device[dev] = p = sym;
    }
    lock.store(0, std::memory_order_release);
    if (!p) { *status = finish_launch(0); if (*status == NMT_OK) *status = NMT_ERR_LAUNCH; return nullptr; }
    *status = NMT_OK;
    return p;
}

int launch_gated_bf16(const void* y, const void* z, const float* w, void* out, int64_t rows, int64_t cols,
                      int64_t group_size, float eps, unsigned int* amax_word, bool* tracked, cudaStream_t st);   // rmsnorm_gated.cu
int validate_gated_bf16(const void* y, const void* z, const float* w, const void* out, int64_t rows, int64_t cols,
                        int64_t group_size);                                                                      // rmsnorm_gated.cu

}  // namespace nmt

extern "C" {

int nmt_rmsnorm_gated_quant_fp8(const void* y, const void* z, const float* w, void* out_bf16, void* out_fp8,
                                float* scale_out, unsigned int* amax_scratch, int64_t rows, int64_t cols,
                                int64_t group_size, float eps, void* stream) {
    using namespace nmt;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // every check first: a rejected call enqueues nothing and leaves the caller's scratch word alone
    int s = validate_gated_bf16(y, z, w, out_bf16, rows, cols, group_size);
    if (s != NMT_OK || rows == 0) return s;
    if (!out_fp8 || !amax_scratch) return NMT_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(out_fp8) & 7u) || !aligned4(amax_scratch) || (scale_out && !aligned4(scale_out))) return NMT_ERR_ALIGN;
    if (cudaMemsetAsync(amax_scratch, 0, sizeof(unsigned int), st) != cudaSuccess) return finish_launch(0);
    bool tracked = false;
    s = launch_gated_bf16(y, z, w, out_bf16, rows, cols, group_size, eps, amax_scratch, &tracked, st);
    if (s != NMT_OK) return s;
    const int64_t nv = rows * cols / 8;
    constexpr int U = 4, B = 256;
    if (!tracked)     // group shape outside the register kernel: take the maximum in a pass of its own
        launch_kernel(amax_kernel<kXfIdentity, U>, ew_grid(nv, B, U), B, 0, st, static_cast<const uint4*>(out_bf16), amax_scratch, nv);
    launch_kernel(quant_kernel<kXfIdentity, U>, ew_grid(nv, B, U), B, 0, st, static_cast<const uint4*>(out_bf16),
                  static_cast<uint2*>(out_fp8), static_cast<const unsigned int*>(amax_scratch), scale_out, nv);
    return finish_launch(tracked ? 1 : 2);
}

int nmt_add_rmsnorm_quant_fp8_static(const void* x, const void* r, const float* w, void* out_res, void* out_fp8,
                                     float* scale_out, int64_t rows, int64_t cols, float eps, void* stream) {
    if (rows > nmt::kStaticMaxRows) return NMT_ERR_TOO_LARGE;     // would not fit the built-in scratch: nothing is launched
    int status = NMT_OK;
    void* scratch = nmt::static_scratch_address(&status);
    if (!scratch) return status;
    // Same two kernels as nmt_add_rmsnorm_quant_fp8, with the built-in array as their workspace.  The launcher
    // zeroes the running-maximum word on the stream before the first kernel; the per-row floats are fully
    // rewritten by the first kernel before the second reads them, so stale contents from an earlier call are
    // never observed.
    return nmt::launch_norm_quant<true>(x, r, w, out_res, out_fp8, scale_out, scratch, rows, cols, eps,
                                        static_cast<cudaStream_t>(stream));
}

int64_t nmt_fp8_workspace_bytes(int64_t rows) {
    if (rows < 0) return -1;
    return 256 + ((rows * 4 + 255) / 256) * 256;
}

int nmt_quantize_fp8(const void* x, void* out_fp8, float* scale_out, unsigned int* amax_scratch, int64_t n, void* stream) {
    return nmt::launch_quant_flat<nmt::kXfIdentity>(x, out_fp8, scale_out, amax_scratch, n, static_cast<cudaStream_t>(stream));
}

int nmt_relu2_quant_fp8(const void* u, void* out_fp8, float* scale_out, unsigned int* amax_scratch, int64_t n, void* stream) {
    return nmt::launch_quant_flat<nmt::kXfRelu2>(u, out_fp8, scale_out, amax_scratch, n, static_cast<cudaStream_t>(stream));
}

int nmt_rmsnorm_quant_fp8(const void* x, const float* w, void* out_fp8, float* scale_out, void* workspace,
                          int64_t rows, int64_t cols, float eps, void* stream) {
    return nmt::launch_norm_quant<false>(x, nullptr, w, nullptr, out_fp8, scale_out, workspace, rows, cols, eps,
                                         static_cast<cudaStream_t>(stream));
}

int nmt_add_rmsnorm_quant_fp8(const void* x, const void* r, const float* w, void* out_res, void* out_fp8,
                              float* scale_out, void* workspace, int64_t rows, int64_t cols, float eps, void* stream) {
    return nmt::launch_norm_quant<true>(x, r, w, out_res, out_fp8, scale_out, workspace, rows, cols, eps,
                                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"
