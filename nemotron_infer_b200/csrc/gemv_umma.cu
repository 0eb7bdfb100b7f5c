// W8A16 GEMV on the 5th-generation tensor cores: tcgen05.mma (kind::f8f6f4) fed by TMA, accumulator in tensor memory.
//
// The mma.sync kernel in gemv_fp8.cu has to turn every e4m3 weight into f16 in registers first (one convert per two
// bytes plus the moves around it: ~75 warp instructions per KB of W) and keeps its bytes in flight in registers; at 16
// warps per SM it is bound by memory latency and instruction issue at 4.0-4.4 TB/s.  Here the weights never enter a
// register and are never converted:
//   * W is described once per call by a 2-D tensor map (rows x K bytes, 128-byte swizzle).  A CTA owns a tile of 128
//     consecutive rows and a contiguous range of K; its producer lane brings the tile in as boxes of 128 rows x 128
//     bytes (16 KB, one cp.async.bulk.tensor each) through a ring in shared memory.  Rows past N and bytes past K are
//     zero-filled by the copy engine, so ragged shapes need no special case.
//   * One lane issues the MMAs: D[128 rows, 16] += A[128 x 32 e4m3] * B[16 x 32 e4m3], four per box, straight from the
//     ring (shared-memory descriptors); the 128 x 16 fp32 accumulator lives in tensor memory (32 columns).  A stage is
//     handed back to the producer by tcgen05.commit on its mbarrier.
//   * The activation side carries the conversion cost, once per CTA instead of once per weight: x (bf16, 8 significant
//     bits) is scaled by a power of two taken from max|x| so that the maximum lands in [128, 256) and split EXACTLY into
//     two e4m3 terms, x * 2^-e = hi + lo / 16 (hi = the top four significant bits, lo = 16 x the remainder), which are
//     rows 0 and 1 of B (the other 14 rows are zero).  Column 0 of D is the hi partial sum, column 1 the lo one; they
//     are recombined in fp32 as D0 + D1 / 16.  Every product is exact and accumulation is fp32.  The split is exact
//     for every element within 2^-12 of the largest; smaller elements are rounded to within 2^-17 * max|x|.
//   * K is split over the CTAs of a thread-block cluster (1, 2, 4 or 8) so that short-and-wide matrices still fill the
//     GPU; the partial sums of a row tile meet in the shared memory of the cluster's first CTA (distributed shared
//     memory stores, one cluster barrier) and are added there in rank order - deterministic, no scratch in global
//     memory, no atomics.
// The ring is filling from the kernel's first cycle: the producer does not wait for the preceding kernel (W is a
// constant of the model, see the ordering contract in nemotron_b200.h) nor for x to be staged.
// Every wait is bounded (nmt_tma.cuh).  A wait that runs out is counted, sets a CTA-wide flag, and everybody skips
// to the end: the producer drains the copies it still has in flight, the cluster barrier is still reached, tensor
// memory is freed, results are void.
#include <cuda.h>
#include <cuda_fp8.h>

#include "nmt_tma.cuh"

namespace nmt {

NMT_DEFINE_TIMEOUT_READER();

constexpr int kUM = 128;                       // rows per tile = MMA M = lanes of tensor memory
constexpr int kUN = 16;                        // MMA N (smallest for M = 128); rows 0 / 1 of B carry x
constexpr int kBoxK = 128;                     // bytes of K per box = one 128-byte swizzle span = four MMAs of K 32
constexpr int kStageBytes = kUM * kBoxK;       // 16 KB
constexpr int kBBoxBytes = kUN * kBoxK;        // 2 KB of B per box of K
constexpr int kUmmaThreads = 192;              // warps 0-3: x staging and epilogue; warp 4: TMA producer; warp 5: MMA issuer
constexpr int kTmemCols = 32;
constexpr int kMaxCluster = 8;

// Instruction descriptor (32 bits): D fp32 (bits 4-5 = 1), A and B e4m3 (bits 7-9, 10-12 = 0), both K-major (bits 15, 16 = 0),
// N / 8 at bits 17-22, M / 16 at bits 24-28.
constexpr uint32_t kIdesc = (1u << 4) | (static_cast<uint32_t>(kUN >> 3) << 17) | (static_cast<uint32_t>(kUM >> 4) << 24);

// Shared-memory matrix descriptor of a K-major operand stored as rows of 128 bytes with the 128-byte swizzle: start
// address / 16 (bits 0-13), leading byte offset / 16 (bits 16-29; unused for this layout, 1), stride byte offset / 16
// (bits 32-45: 8 rows x 128 bytes = 1024 between 8-row groups), descriptor version 1 (bits 46-47), layout type
// SWIZZLE_128B = 2 (bits 61-63).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t da, uint64_t db, bool accumulate) {
    asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(kIdesc), "r"(static_cast<uint32_t>(accumulate)) : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has finished (reading shared memory included).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tma_box_load(void* smem_dst, const CUtensorMap* map, int k_byte, int row, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(k_byte), "r"(row), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_f32(float* local_ptr, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Two fp32 values -> two e4m3 bytes (`lo` in the low byte), round to nearest, saturating.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
    uint32_t r;
    asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

struct UmmaFusion {
    const float* norm_w;          // non-null: x = rmsnorm(x) * norm_w first
    float eps, inv_cols;
    int norm_threads;             // threads per row of the stand-alone norm kernel (its summation order)
    int activation;               // 1: y = relu(y)^2
    const uint16_t* residual;     // non-null: y += residual[row]
};

__global__ void __launch_bounds__(kUmmaThreads, 1)
gemv_w8a16_umma_kernel(const __grid_constant__ CUtensorMap wmap, const __nv_bfloat16* __restrict__ x, const float* __restrict__ w_scale,
                       __nv_bfloat16* __restrict__ y, int N, int K, int kparts, int stages, UmmaFusion fu) {
    extern __shared__ __align__(1024) uint8_t smem_u[];
    __shared__ uint64_t s_full[12], s_empty[12], s_xready, s_done;
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    __shared__ float s_red[8];
    __shared__ float s_part[kMaxCluster][kUM];                    // partial sums of the cluster's CTAs (used in rank 0)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t rank = kparts > 1 ? cluster_rank() : 0u;
    const int tile = blockIdx.x / kparts;
    const int boxes_total = (K + kBoxK - 1) / kBoxK;
    const int base = boxes_total / kparts, rem = boxes_total % kparts;
    const int box0 = static_cast<int>(rank) * base + min(static_cast<int>(rank), rem);
    const int nbox = base + (static_cast<int>(rank) < rem ? 1 : 0);        // boxes of K this CTA multiplies
    // shared memory: [ring: stages x 16 KB][B: nbox_max x 2 KB][normalised x: K bf16 (fused form only)]; the swizzled tiles
    // need 1024-byte alignment in the shared-memory window, which the launcher leaves room for
    uint8_t* ring = smem_u + ((1024u - (smem_u32(smem_u) & 1023u)) & 1023u);
    uint8_t* bx = ring + (size_t)stages * kStageBytes;
    const int nbox_max = base + (rem ? 1 : 0);
    uint4* xn = reinterpret_cast<uint4*>(bx + (size_t)nbox_max * kBBoxBytes);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], 1); }
        mbar_init(&s_xready, 1);
        mbar_init(&s_done, 1);
        s_abort = 0;
        mbar_init_fence();
    }
    if (warp == 0) {                                               // tensor memory: 32 columns for the 128 x 16 fp32 accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(&s_tmem);
    int issued = 0;                                                // producer lane: boxes whose copy has been issued

    if (warp == 4) {
        // ---------------- producer ----------------
        if (lane == 0) {
            bool ok = true;
            for (int n = 0; n < nbox && ok; ++n) {
                const int s = n % stages;
                if (n >= stages) ok = mbar_wait(&s_empty[s], static_cast<uint32_t>(n / stages - 1) & 1u);
                if (!ok) break;
                mbar_arrive_expect_tx(&s_full[s], kStageBytes);
                tma_box_load(ring + (size_t)s * kStageBytes, &wmap, (box0 + n) * kBoxK, tile * kUM, &s_full[s]);
                issued = n + 1;
            }
            pdl_trigger();                                         // every copy of this CTA has been issued
            if (!ok) atomicExch(&s_abort, 1);
        }
    } else if (warp == 5) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            bool ok = mbar_wait(&s_xready, 0);
            for (int n = 0; n < nbox && ok; ++n) {
                const int s = n % stages;
                ok = mbar_wait(&s_full[s], static_cast<uint32_t>(n / stages) & 1u);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a0 = smem_u32(ring + (size_t)s * kStageBytes), b0 = smem_u32(bx + (size_t)n * kBBoxBytes);
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)                     // K = 32 bytes per MMA: advance both descriptors inside the swizzle span
                    umma_f8(tmem, umma_desc(a0 + kk * 32), umma_desc(b0 + kk * 32), n > 0 || kk > 0);
                umma_commit(&s_empty[s]);                          // the stage is free once these MMAs have read it
            }
            if (ok) umma_commit(&s_done);                          // accumulator complete
            else atomicExch(&s_abort, 1);
        }
    } else {
        // ---------------- warps 0-3: stage x, then the epilogue ----------------
        pdl_wait();                                                // x (and the residual) may come from the preceding kernel
        const int nv = K / 8;
        const uint4* xv = reinterpret_cast<const uint4*>(x);
        const bool normed = fu.norm_w != nullptr;
        if (normed) {
            // the stand-alone kernel's shape (rmsnorm_ctarow_kernel, one row): thread t of norm_threads owns vectors t, t + nt, ...
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
            epilogue_barrier();
            if (threadIdx.x < nt) {
                float total = 0.f;
                for (int i = 0; i < nt / 32; ++i) total += s_red[i];
                const float rstd = rsqrtf(total * fu.inv_cols + fu.eps);
#pragma unroll 2
                for (int v = threadIdx.x; v < nv; v += nt) {
                    float2 pr[4];
                    unpack8x2(ld_stream(xv + v), pr);
                    xn[v] = scale8(pr, rstd, ld_weight4(fu.norm_w + (size_t)v * 8), ld_weight4(fu.norm_w + (size_t)v * 8 + 4));
                }
            }
            epilogue_barrier();
        }
        const uint4* src = normed ? xn : xv;
        float m = 0.f;
#pragma unroll 2
        for (int v = threadIdx.x; v < nv; v += 128) {
            const uint4 u = normed ? src[v] : __ldg(src + v);
            const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) m = fmaxf(m, fmaxf(fabsf(bf16_lo(w4[k])), fabsf(bf16_hi(w4[k]))));
        }
        m = warp_max(m);
        if (lane == 0) s_red[4 + warp] = m;
        epilogue_barrier();
        const float mm = fmaxf(fmaxf(s_red[4], s_red[5]), fmaxf(s_red[6], s_red[7]));
        int e = 0;
        if (mm > 0.f && mm < 3.0e38f) e = static_cast<int>((__float_as_uint(mm) >> 23) & 0xff) - 127 - 7;   // max|x| lands in [2^7, 2^8)
        e = max(e, -120);                                          // keeps 2^-e and 2^e normal fp32 numbers
        const float down = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);      // 2^-e
        // B for this CTA's boxes of K: per box 16 rows x 128 bytes in the 128-byte-swizzled K-major layout (the 16-byte unit
        // u of row r sits at unit u ^ (r & 7)); row 0 = hi, row 1 = lo, rows 2-15 = 0.  A vector of 8 bf16 is 8 bytes of a plane.
        for (int i = threadIdx.x; i < nbox * (kBBoxBytes / 16); i += 128) {            // zero fill, rows 2-15 included
            reinterpret_cast<uint4*>(bx)[i] = make_uint4(0, 0, 0, 0);
        }
        epilogue_barrier();
        const int v_lo = box0 * (kBoxK / 8), v_hi = min(nv, (box0 + nbox) * (kBoxK / 8));
        for (int v = v_lo + threadIdx.x; v < v_hi; v += 128) {
            const uint4 u = normed ? src[v] : __ldg(src + v);
            const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
            uint32_t h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float x0 = bf16_lo(w4[k]) * down, x1 = bf16_hi(w4[k]) * down;
                const float h0 = __uint_as_float(__float_as_uint(x0) & 0xfff00000u), h1 = __uint_as_float(__float_as_uint(x1) & 0xfff00000u);
                h[k] = f32x2_to_e4m3x2(h0, h1);
                l[k] = f32x2_to_e4m3x2((x0 - h0) * 16.f, (x1 - h1) * 16.f);
            }
            const int kbyte = (v - v_lo) * 8;                      // byte offset of these 8 elements inside this CTA's K range
            const int box = kbyte / kBoxK, inbox = kbyte % kBoxK, unit = inbox / 16, off = inbox % 16;
            uint8_t* bb = bx + (size_t)box * kBBoxBytes;
            *reinterpret_cast<uint2*>(bb + 0 * 128 + ((unit ^ 0) * 16) + off) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
            *reinterpret_cast<uint2*>(bb + 1 * 128 + ((unit ^ 1) * 16) + off) = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
        }
        fence_proxy_async_smem();                                  // generic-proxy writes -> visible to the tensor core's reads
        epilogue_barrier();
        if (threadIdx.x == 0) mbar_arrive(&s_xready);

        // ---- epilogue: D[row][0] + D[row][1] / 16 ----
        bool ok = mbar_wait(&s_done, 0);
        if (*reinterpret_cast<volatile int*>(&s_abort) != 0) ok = false;
        ok = __all_sync(0xffffffffu, ok);                          // the tensor-memory load below is warp-wide
        float partial = 0.f;
        if (ok) {
            tc_fence_after();
            uint32_t d0, d1;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(d0), "=r"(d1) : "r"(tmem + (static_cast<uint32_t>(warp * 32) << 16)));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            partial = __uint_as_float(d0) + __uint_as_float(d1) * 0.0625f;
        } else if (threadIdx.x == 0) {
            atomicExch(&s_abort, 1);
        }
        if (kparts > 1 && rank != 0) st_cluster_f32(&s_part[rank][threadIdx.x], 0, partial);
        else s_part[0][threadIdx.x] = partial;
    }
    // Everybody meets here: partial sums are in the first CTA's shared memory once the cluster barrier is passed.
    if (kparts > 1) cluster_sync_all(); else __syncthreads();
    if (warp < 4 && rank == 0) {
        const int row = tile * kUM + threadIdx.x;
        if (row < N) {
            float sum = s_part[0][threadIdx.x];
            for (int r = 1; r < kparts; ++r) sum += s_part[r][threadIdx.x];
            // the exponent is recomputed by every CTA from the same x, so rank 0's is everybody's
            const float mm = fmaxf(fmaxf(s_red[4], s_red[5]), fmaxf(s_red[6], s_red[7]));
            int e = 0;
            if (mm > 0.f && mm < 3.0e38f) e = static_cast<int>((__float_as_uint(mm) >> 23) & 0xff) - 127 - 7;
            e = max(e, -120);
            const float up = __uint_as_float(static_cast<uint32_t>(127 + e) << 23);     // 2^e
            uint32_t yb = pack_bf16x2((sum * up) * __ldg(w_scale + row), 0.f);
            if (fu.activation == 1) yb = relu2_bf16x2(yb);
            if (fu.residual) yb = add_bf16x2_rn(static_cast<uint32_t>(fu.residual[row]), yb);
            reinterpret_cast<uint16_t*>(y)[row] = static_cast<uint16_t>(yb & 0xffffu);
        }
    }
    // A wait ran out somewhere in this CTA (counted; results void): copies may still be in flight - the producer lane
    // waits, bounded again, for the last fill of every stage before the CTA gives up its shared memory.
    if (warp == 4 && lane == 0 && *reinterpret_cast<volatile int*>(&s_abort) != 0) {
        for (int n = max(0, issued - stages); n < issued; ++n) mbar_wait(&s_full[n % stages], static_cast<uint32_t>(n / stages) & 1u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    pdl_trigger();
}

// ---------------------------------------------------------------------------------------------
// Host side: the tensor map of W (driver entry point fetched at run time; the library does not link libcuda).
// ---------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int launch_gemv_umma(const void* x, const float* norm_w, float eps, const void* W, const float* w_scale, int activation,
                     const void* residual, void* y, int N, int K, cudaStream_t st) {
    if ((K % 64) != 0 || K > 16384 || (reinterpret_cast<uintptr_t>(x) & 15u)) return NMT_ERR_UNSUPPORTED;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return NMT_ERR_UNSUPPORTED;
    // one map per (W, N, K); a small per-thread cache saves the encode for the weights a decode loop keeps calling with
    struct Entry { const void* W; int N, K; CUtensorMap map; };
    static thread_local Entry cache[64];
    static thread_local int cache_n = 0, cache_next = 0;
    const CUtensorMap* map = nullptr;
    for (int i = 0; i < cache_n; ++i) if (cache[i].W == W && cache[i].N == N && cache[i].K == K) { map = &cache[i].map; break; }
    if (!map) {
        Entry& en = cache[cache_next];
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(N)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K)};
        const cuuint32_t box[2] = {kBoxK, kUM};
        const cuuint32_t estr[2] = {1, 1};
        if (encode(&en.map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(W), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return NMT_ERR_UNSUPPORTED;
        en.W = W; en.N = N; en.K = K;
        map = &en.map;
        cache_next = (cache_next + 1) % 64;
        if (cache_n < 64) ++cache_n;
    }
    const int tiles = (N + kUM - 1) / kUM;
    const int boxes = (K + kBoxK - 1) / kBoxK;
    // K parts (= cluster size): enough CTAs for about two per SM, a power of two, never more than there are boxes
    int kparts = tune("gemv.kparts", 0);
    if (kparts != 1 && kparts != 2 && kparts != 4 && kparts != 8) {
        kparts = 1;
        while (kparts < kMaxCluster && tiles * kparts * 2 <= 2 * kSmCount && kparts * 2 <= boxes) kparts *= 2;
    }
    while (kparts > 1 && kparts > boxes) kparts /= 2;
    const int nbox_max = (boxes + kparts - 1) / kparts;
    int stages = tune("gemv.ring_stages", 4);            // 4 x 16 KB in flight per CTA, two CTAs per SM
    if (stages > 12) stages = 12;
    if (stages > nbox_max) stages = nbox_max;
    if (stages < 1) stages = 1;
    const size_t smem = (size_t)stages * kStageBytes + (size_t)nbox_max * kBBoxBytes + (norm_w ? (size_t)K * 2 : 0) + 1024;
    if (smem > 200 * 1024) return NMT_ERR_UNSUPPORTED;
    UmmaFusion fu = {};
    fu.norm_w = norm_w;
    fu.eps = eps;
    fu.inv_cols = 1.0f / static_cast<float>(K);
    fu.norm_threads = default_norm_block(K / 8, false);
    fu.activation = activation;
    fu.residual = static_cast<const uint16_t*>(residual);
    if (norm_w && fu.norm_threads > 128) return NMT_ERR_UNSUPPORTED;     // the prologue runs on the four staging warps
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        if (cudaFuncSetAttribute(gemv_w8a16_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess) return finish_launch(0);
        configured[dev] = true;
    }
    launch_cluster_kernel(gemv_w8a16_umma_kernel, tiles * kparts, kparts, kUmmaThreads, smem, st, *map, static_cast<const __nv_bfloat16*>(x),
                          w_scale, static_cast<__nv_bfloat16*>(y), N, K, kparts, stages, fu);
    return finish_launch(1);
}

}  // namespace nmt
