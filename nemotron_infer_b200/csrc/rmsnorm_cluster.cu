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

#include "nmt_common.cuh"

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

// Returns NMT_ERR_UNSUPPORTED when the row does not fit a cluster of 8 (more than 262,144 bf16) or `cluster`
// is not 2, 4 or 8.  cluster = 0 picks 2 where two CTAs can hold the row in 8 vectors per thread, else 8.
int launch_norm_cluster(bool fuse, const void* x, const void* r, const float* w, void* out_res, void* out,
                        int64_t rows, int64_t cols, float eps, int cluster, cudaStream_t st) {
    const int64_t nv64 = cols / 8;
    if (nv64 > (int64_t)kClusterMax * kClusterBlockMax * 8) return NMT_ERR_UNSUPPORTED;
    const int nv = static_cast<int>(nv64);
    const int block = tune("norm.cluster_block", 512) == 256 ? 256 : 512;
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
