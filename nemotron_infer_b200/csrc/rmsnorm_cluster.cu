// RMSNorm (optionally fused with the residual add) for rows too wide for one CTA's registers.
//
// A thread-block cluster of C CTAs owns one row at a time: CTA r of the cluster keeps vectors
// [r * per_cta, (r + 1) * per_cta) of the row in registers, reduces its share of the sum of squares with warp
// shuffles and a shared-memory step, and then writes that partial sum into slot r of EVERY CTA of the cluster
// through distributed shared memory.  One hardware cluster barrier later each CTA adds the C partial sums in
// rank order (so every CTA gets the same bits), scales its share and stores it.  Each activation byte crosses
// HBM once: read x (and r), write out (and out_res) - where the single-CTA kernels stop (more than 8 vectors per
// thread at 512 threads, i.e. rows wider than 32,768 bf16), the alternative is a second read of the row.
//
// The partial-sum slots are double-buffered by row parity, which makes one barrier per row enough: a CTA can be
// at most one row ahead of the slowest CTA of its cluster, because it cannot pass row i+1's barrier before that
// CTA has arrived there, i.e. has finished reading row i's slots.  A final barrier keeps every CTA's shared
// memory alive until its peers' last remote writes have landed.
#include <cooperative_groups.h>

#include "nmt_tma.cuh"

namespace cg = cooperative_groups;

namespace nmt {

constexpr int kClusterBlockMax = 512;
constexpr int kClusterMax = 8;        // portable cluster size limit

template <int SLOTS, int BLOCK, bool FUSE_ADD>
__global__ void __launch_bounds__(BLOCK)
rmsnorm_cluster_kernel(const uint4* x, const uint4* r, const float* __restrict__ w, uint4* out_res, uint4* out,
                       int64_t rows, int nv, int per_cta, float inv_cols, float eps) {
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = static_cast<int>(cluster.num_blocks());
    const int crank = static_cast<int>(cluster.block_rank());
    constexpr int kClusterBlock = BLOCK;
    __shared__ float s_warp[kClusterBlock / 32];
    __shared__ float s_part[2][kClusterMax];                      // [row parity][cluster rank]
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int v0 = crank * per_cta;                               // this CTA's share of the row
    const int vend = min(nv, v0 + per_cta);
    const int64_t cluster_id = blockIdx.x / csize, nclusters = gridDim.x / csize;
    int flip = 0;
#pragma unroll 1
    for (int64_t row = cluster_id; row < rows; row += nclusters, flip ^= 1) {   // same trip count for every CTA of a cluster
        uint4 a[SLOTS], b[SLOTS];
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int v = v0 + s * kClusterBlock + threadIdx.x;
            if (v < vend) {
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
                a[s] = add_bf16x8_rn(a[s], b[s]);                 // the norm sees the bf16 value the next block reads back
                // Stored now, not after the barrier: measured 20 % faster, the write overlaps the reduction.
                const int v = v0 + s * kClusterBlock + threadIdx.x;
                if (v < vend) st_stream(out_res + row * nv + v, a[s]);
            }
            float2 p[4];
            unpack8x2(a[s], p);
#pragma unroll
            for (int k = 0; k < 4; ++k) acc = __ffma2_rn(p[k], p[k], acc);
        }
        const float ss = warp_sum(acc.x + acc.y);
        if (lane == 0) s_warp[wid] = ss;
        __syncthreads();
        if (wid == 0) {
            float t = lane < kClusterBlock / 32 ? s_warp[lane] : 0.f;
            t = warp_sum(t);
            // lane i delivers this CTA's partial sum to CTA i of the cluster
            if (lane < csize) *cluster.map_shared_rank(&s_part[flip][crank], lane) = t;
        }
        cluster.sync();                                           // remote writes are visible after this barrier
        float total = 0.f;
        for (int i = 0; i < csize; ++i) total += s_part[flip][i];
        const float rstd = rsqrtf(total * inv_cols + eps);
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int v = v0 + s * kClusterBlock + threadIdx.x;
            if (v < vend) {
                float2 p[4];
                unpack8x2(a[s], p);
                st_stream(out + row * nv + v, scale8(p, rstd, ld_weight4(w + (size_t)v * 8), ld_weight4(w + (size_t)v * 8 + 4)));
            }
        }
    }
    cluster.sync();
    pdl_trigger();
}

// ---------------------------------------------------------------------------------------------
// Staged form: bytes in flight live in shared memory, not in registers.
//
// The kernel above keeps a CTA's loads in registers: one 512-thread CTA per SM at the register limit has 64 KB
// (plain) to 128 KB (fused) in flight, which is what holds it at 4 - 6 TB/s.  Here every CTA owns a ring of
// STAGES row shares in shared memory.  A row share is one contiguous 16-byte-aligned range of the row, so one
// elected thread moves it with ONE bulk copy per input that completes on an mbarrier; up to ~190 KB per SM are
// in flight while the 512 threads work on the shares that have landed: they reduce a share where it lies,
// exchange the partial sums with the other CTAs of the cluster by st.async (a store into a peer's shared memory
// that counts bytes on an mbarrier there), scale the share out of the stage and only then hand the stage back to
// the producer.  No cluster barrier inside the loop; every wait is a bounded poll of an mbarrier in this CTA's
// own shared memory.  A row is done in two halves - sum of squares and send, then receive and scale - and row
// i+1's first half runs before row i's second, so the exchange is off the critical path.  That lets a CTA
// send row i+1 while a peer still sits before its second half of row i-2 (this CTA needed only the peer's row i-1
// partial sum to get here), hence four partial-sum slots and barriers, indexed by row % 4.
// ---------------------------------------------------------------------------------------------
NMT_DEFINE_TIMEOUT_READER();

constexpr int kStagedBlock = 512;
constexpr int kStagedMaxStages = 4;
constexpr int kPartSlots = 4;          // partial-sum slots: rows i-2 .. i+1 can be in use at the same time (see above)
constexpr size_t kStagedSmemBudget = 200 * 1024;

__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, int rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_async_f32(uint32_t remote_data, float v, uint32_t remote_bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(remote_data), "r"(__float_as_uint(v)), "r"(remote_bar) : "memory");
}

template <int SLOTS, bool FUSE_ADD>
__global__ void __launch_bounds__(kStagedBlock, 1)               // the ring leaves room for one CTA per SM: registers are free
rmsnorm_cluster_staged_kernel(const uint4* x, const uint4* r, const float* __restrict__ w, uint4* out_res, uint4* out,
                              int64_t rows, int nv, int per_cta, float inv_cols, float eps, int stages) {
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    const int csize = static_cast<int>(cluster.num_blocks());
    const int crank = static_cast<int>(cluster.block_rank());
    extern __shared__ __align__(128) uint8_t ring[];              // [stages][x share | r share]
    __shared__ float s_warp[kStagedBlock / 32];
    __shared__ __align__(16) float s_part[kPartSlots][kClusterMax];   // [row % 4][cluster rank]
    __shared__ __align__(8) uint64_t s_pbar[kPartSlots];         // partial sums of a row have arrived
    __shared__ __align__(8) uint64_t s_full[kStagedMaxStages];   // a stage's bulk copies have landed
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int v0 = crank * per_cta, vend = min(nv, v0 + per_cta);
    const int nmine = max(vend - v0, 0);                          // vectors of this CTA's share
    const uint32_t share_bytes = static_cast<uint32_t>(per_cta) * 16u;
    const uint32_t stage_bytes = share_bytes * (FUSE_ADD ? 2u : 1u);
    const uint32_t copy_bytes = static_cast<uint32_t>(nmine) * 16u;
    const int64_t cluster_id = blockIdx.x / csize, nclusters = gridDim.x / csize;
    const int64_t my_rows = cluster_id < rows ? (rows - cluster_id + nclusters - 1) / nclusters : 0;   // same for the whole cluster

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPartSlots; ++s) mbar_init(&s_pbar[s], 1);
        for (int s = 0; s < stages; ++s) mbar_init(&s_full[s], 1);
        mbar_init_fence();
    }
    cluster.sync();                                               // every CTA's barriers exist before anyone sends

    // Producer side (thread 0): fill stage (i % stages) with this CTA's share of its i-th row.
    auto fill = [&](int64_t i) {
        const int s = static_cast<int>(i % stages);
        const int64_t row = cluster_id + i * nclusters;
        uint8_t* dst = ring + (size_t)s * stage_bytes;
        if (copy_bytes) {
            mbar_arrive_expect_tx(&s_full[s], FUSE_ADD ? 2 * copy_bytes : copy_bytes);
            bulk_load(dst, x + row * nv + v0, copy_bytes, &s_full[s]);
            if (FUSE_ADD) bulk_load(dst + share_bytes, r + row * nv + v0, copy_bytes, &s_full[s]);
        } else {
            mbar_arrive(&s_full[s]);                              // a CTA with an empty share still keeps the phases in step
        }
    };
    int64_t issued = 0;                                           // thread 0 only
    if (threadIdx.x == 0)
        for (; issued < my_rows && issued < stages; ++issued) fill(issued);

    // A thread owns the same columns of every row, so its norm weights are loaded once and stay in registers: a wide
    // row's weights (4 bytes per column, twice the activation bytes) fit no L1 next to the ring, and fetching them
    // from L2 inside the second half of every row was what that half spent its time waiting for.
    float4 wreg[SLOTS][2];
#pragma unroll
    for (int q = 0; q < SLOTS; ++q) {
        const int v = q * kStagedBlock + threadIdx.x;
        const size_t col = (size_t)(v0 + (v < nmine ? v : 0)) * 8;
        wreg[q][0] = nmine > 0 ? ld_weight4(w + col) : make_float4(0.f, 0.f, 0.f, 0.f);
        wreg[q][1] = nmine > 0 ? ld_weight4(w + col + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    bool ok = true;
    // First half of a row: the landed share -> sum of squares (the fused form also forms x + r, stores it as out_res and
    // leaves it in the stage for the second half), then this CTA's partial sum goes out to every CTA of the cluster.
    auto first_half = [&](int64_t i) {
        const int s = static_cast<int>(i % stages);
        const int64_t row = cluster_id + i * nclusters;
        // A wait that runs out is counted and ends this CTA's work (its peers then run out of patience the same way);
        // the vote keeps the exit block-uniform, so that nobody is left alone at a block barrier.
        ok = __syncthreads_and(mbar_wait(&s_full[s], static_cast<uint32_t>(i / stages) & 1u));
        if (!ok) return;
        uint4* sx = reinterpret_cast<uint4*>(ring + (size_t)s * stage_bytes);
        const uint4* sr = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes + share_bytes);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int v = q * kStagedBlock + threadIdx.x;
            if (v < nmine) {
                uint4 a = lds128(sx + v);
                if (FUSE_ADD) {
                    a = add_bf16x8_rn(a, lds128(sr + v));
                    sx[v] = a;
                    st_stream(out_res + row * nv + v0 + v, a);
                }
                float2 p[4];
                unpack8x2(a, p);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc = __ffma2_rn(p[k], p[k], acc);
            }
        }
        const float ss = warp_sum(acc.x + acc.y);
        if (lane == 0) s_warp[wid] = ss;
        __syncthreads();
        if (wid == 0) {
            const int slot = static_cast<int>(i & (kPartSlots - 1));
            float t = lane < kStagedBlock / 32 ? s_warp[lane] : 0.f;
            t = warp_sum(t);
            if (lane == 0) mbar_arrive_expect_tx(&s_pbar[slot], static_cast<uint32_t>(csize) * 4u);
            if (lane < csize)                                     // lane j delivers this CTA's partial sum to CTA j
                st_async_f32(map_to_rank(smem_u32(&s_part[slot][crank]), lane), t, map_to_rank(smem_u32(&s_pbar[slot]), lane));
        }
    };
    // Second half: all partial sums of the row are here -> scale the share out of the stage, then hand the stage back.
    auto second_half = [&](int64_t i) {
        const int s = static_cast<int>(i % stages);
        const int slot = static_cast<int>(i & (kPartSlots - 1));
        const int64_t row = cluster_id + i * nclusters;
        ok = __syncthreads_and(mbar_wait(&s_pbar[slot], static_cast<uint32_t>(i / kPartSlots) & 1u));
        if (!ok) return;
        float total = 0.f;
        for (int j = 0; j < csize; ++j) total += s_part[slot][j];
        const float rstd = rsqrtf(total * inv_cols + eps);
        const uint4* sx = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
#pragma unroll
        for (int q = 0; q < SLOTS; ++q) {
            const int v = q * kStagedBlock + threadIdx.x;
            if (v < nmine) {
                float2 p[4];
                unpack8x2(lds128(sx + v), p);
                st_stream(out + row * nv + v0 + v, scale8(p, rstd, wreg[q][0], wreg[q][1]));
            }
        }
        fence_proxy_async_smem();                                 // this thread's accesses to the stage come before its refill
        __syncthreads();
        if (threadIdx.x == 0 && issued < my_rows) fill(issued++); // the stage is free again: next row share on its way
    };
    // Row i+1's first half runs while row i's partial sums are still travelling.
    int64_t done = 0;                                             // rows whose second half is complete
    if (my_rows > 0) first_half(0);
#pragma unroll 1
    for (int64_t i = 0; i < my_rows && ok; ++i) {
        if (i + 1 < my_rows) first_half(i + 1);
        if (!ok) break;
        second_half(i);
        if (ok) done = i + 1;
    }
    // A wait ran out (counted; the results are void): do not leave while bulk copies into this CTA's shared memory
    // may still be in flight - wait, bounded again, for every stage that was filled and not handed back.
    if (!ok && threadIdx.x == 0) {
        for (int64_t j = done; j < issued; ++j)
            mbar_wait(&s_full[static_cast<int>(j % stages)], static_cast<uint32_t>(j / stages) & 1u);
    }
    cluster.sync();                                               // nobody leaves while a peer may still write to it
    pdl_trigger();
}

// Resident clusters of the staged kernel (asked of the runtime once per kernel, cluster size, stage count and device).
template <typename K>
static int staged_resident_clusters(K kern, int cluster, size_t smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(cluster * kSmCount));
    cfg.blockDim = dim3(kStagedBlock);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(cluster);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = kSmCount / cluster / 2;                                // conservative
    }
    return n;
}

template <int SLOTS, bool FUSE_ADD>
static int launch_staged(const void* x, const void* r, const float* w, void* out_res, void* out, int64_t rows, int nv,
                         int cluster, int per_cta, int stages, float inv_cols, float eps, cudaStream_t st) {
    auto kern = rmsnorm_cluster_staged_kernel<SLOTS, FUSE_ADD>;
    const size_t smem = (size_t)stages * per_cta * 16 * (FUSE_ADD ? 2 : 1);
    static bool configured[64] = {};
    static int resident[64][9][kStagedMaxStages + 1] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return NMT_ERR_UNSUPPORTED;
    if (!configured[dev]) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kStagedSmemBudget)) != cudaSuccess)
            return finish_launch(0);
        configured[dev] = true;
    }
    // per (cluster, stages) the shared-memory footprint is bounded by the budget, so the first query's answer is
    // reused for every width that maps to the same pair
    if (resident[dev][cluster][stages] <= 0) resident[dev][cluster][stages] = staged_resident_clusters(kern, cluster, kStagedSmemBudget);
    int64_t ncl = resident[dev][cluster][stages];
    if (ncl > rows) ncl = rows;
    if (ncl < 1) ncl = 1;
    launch_cluster_kernel(kern, static_cast<int>(ncl) * cluster, cluster, kStagedBlock, smem, st, static_cast<const uint4*>(x),
                          static_cast<const uint4*>(r), w, static_cast<uint4*>(out_res), static_cast<uint4*>(out), rows, nv, per_cta,
                          inv_cols, eps, stages);
    return finish_launch(1);
}

// Staged form if some cluster size gives at least two stages within the shared-memory budget; else NMT_ERR_UNSUPPORTED.
// cluster = 0: smallest of 2 / 4 / 8 that fits; 1: a single CTA per row (the ring without the exchange partners).
static int launch_norm_cluster_staged(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                                      int64_t rows, int nv, float inv_cols, float eps, int cluster, cudaStream_t st) {
    // The smallest cluster whose share gives a ring of at least two stages: measured, a smaller cluster with a
    // shallower ring beats a larger one with a deeper ring every time (e.g. 476 vs 507 us at 8192 x 40,000 fused).
    int best_c = 0, best_stages = 0;
    for (int c = (cluster == 1 ? 1 : 2); c <= kClusterMax && best_c == 0; c *= 2) {
        if (cluster >= 1 && c != cluster) continue;
        const int pc = (nv + c - 1) / c;
        if ((pc + kStagedBlock - 1) / kStagedBlock > 8) continue;     // a thread keeps its columns' weights in registers
        const size_t stage = (size_t)pc * 16 * (fuse ? 2 : 1);
        int stages = static_cast<int>(kStagedSmemBudget / stage);
        if (stages > kStagedMaxStages) stages = kStagedMaxStages;
        if (stages < 2) continue;
        best_c = c;
        best_stages = stages;
    }
    if (best_c == 0) return NMT_ERR_UNSUPPORTED;
    const int forced_stages = tune("norm.cluster_stages", 0);
    if (forced_stages >= 2 && forced_stages <= best_stages) best_stages = forced_stages;
    const int pc = (nv + best_c - 1) / best_c;
    const int slots = (pc + kStagedBlock - 1) / kStagedBlock;
#define NMT_STAGED_CASE(S)                                                                                                   \
    return fuse ? launch_staged<S, true>(x, r, w, out_res, out, rows, nv, best_c, pc, best_stages, inv_cols, eps, st)       \
                : launch_staged<S, false>(x, r, w, out_res, out, rows, nv, best_c, pc, best_stages, inv_cols, eps, st)
    if (slots <= 1) NMT_STAGED_CASE(1);
    if (slots <= 2) NMT_STAGED_CASE(2);
    if (slots <= 4) NMT_STAGED_CASE(4);
    if (slots <= 6) NMT_STAGED_CASE(6);
    NMT_STAGED_CASE(8);
#undef NMT_STAGED_CASE
}

// One CTA per row with the row staged in shared memory: for rows that fit one CTA's registers only at 6 - 8 vectors
// per thread (20,480 - 32,768 columns), where the register kernel has too few bytes in flight
// (plain norm at 32,768 columns: 6.2 vs 4.7 TB/s; with the residual add the register kernel stays ahead).
int launch_norm_staged_single(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                              int64_t rows, int64_t cols, float eps, cudaStream_t st) {
    const int64_t nv = cols / 8;
    if (nv > 8 * kStagedBlock) return NMT_ERR_UNSUPPORTED;
    return launch_norm_cluster_staged(fuse, x, r, w, out_res, out, rows, static_cast<int>(nv), 1.0f / static_cast<float>(cols), eps, 1, st);
}

// Returns NMT_ERR_UNSUPPORTED when the row does not fit a cluster of 8 (more than 262,144 bf16) or `cluster`
// is not 2, 4 or 8.  cluster = 0 picks 2 where two CTAs can hold the row in 8 vectors per thread, else 8.
int launch_norm_cluster(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                        int64_t rows, int64_t cols, float eps, int cluster, cudaStream_t st) {
    const int64_t nv64 = cols / 8;
    if (nv64 > (int64_t)kClusterMax * kClusterBlockMax * 8) return NMT_ERR_UNSUPPORTED;
    const int nv = static_cast<int>(nv64);
    const int block = tune("norm.cluster_block", 512) == 256 ? 256 : 512;
    if (tune("norm.cluster_staged", 1) == 1) {                     // 1 (default) = shared-memory ring, 2 = registers only
        const int st_status = launch_norm_cluster_staged(fuse, x, r, w, out_res, out, rows, nv, 1.0f / static_cast<float>(cols), eps, cluster, st);
        if (st_status != NMT_ERR_UNSUPPORTED) return st_status;
    }
    if (cluster == 0) cluster = (nv + 1) / 2 <= block * 8 ? 2 : 8;   // measured: 4 is never the fastest
    if (cluster != 2 && cluster != 4 && cluster != 8) return NMT_ERR_UNSUPPORTED;
    const int per_cta = (nv + cluster - 1) / cluster;
    const int slots = (per_cta + block - 1) / block;
    if (slots > 8) return NMT_ERR_UNSUPPORTED;
    // one cluster per row up to about three CTAs per SM (the surplus queues, which the scheduler fills gaps with), then rows are strided
    int64_t nclusters = rows;
    const int64_t cap = (int64_t)kSmCount * tune("norm.cluster_ctas_per_sm", 3) / cluster;
    if (nclusters > cap) nclusters = cap;
    const int grid = static_cast<int>(nclusters) * cluster;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    auto X = static_cast<const uint4*>(x);
    auto R = static_cast<const uint4*>(r);
    auto OR = static_cast<uint4*>(out_res);
    auto O = static_cast<uint4*>(out);
#define NMT_CLUSTER_LAUNCH(S, B, F) launch_cluster_kernel(rmsnorm_cluster_kernel<S, B, F>, grid, cluster, B, 0, st, X, R, w, OR, O, rows, nv, per_cta, inv_cols, eps)
#define NMT_CLUSTER_CASE(S)                                                  \
    do {                                                                     \
        if (block == 256) { if (fuse) NMT_CLUSTER_LAUNCH(S, 256, true); else NMT_CLUSTER_LAUNCH(S, 256, false); } \
        else { if (fuse) NMT_CLUSTER_LAUNCH(S, 512, true); else NMT_CLUSTER_LAUNCH(S, 512, false); }              \
    } while (0)
    if (slots <= 1) NMT_CLUSTER_CASE(1);
    else if (slots <= 2) NMT_CLUSTER_CASE(2);
    else if (slots <= 3) NMT_CLUSTER_CASE(3);
    else if (slots <= 4) NMT_CLUSTER_CASE(4);
    else if (slots <= 5) NMT_CLUSTER_CASE(5);
    else if (slots <= 6) NMT_CLUSTER_CASE(6);
    else NMT_CLUSTER_CASE(8);
#undef NMT_CLUSTER_CASE
#undef NMT_CLUSTER_LAUNCH
    return finish_launch(1);
}

}  // namespace nmt
