// Mamba-2 state-space recurrence, one token: the step between the conv step and the gated norm of the decode block
// (model/mamba_block.cuh:298-301, 499-502; replaces ops/mamba2/ssm.cuh:43-103, ssm_decode_bf16).
//
//   dt' = clamp(softplus(dt[h] + dt_bias[h]))        dA = exp(-exp(A_log[h]) * dt')
//   state[h, p, n] = state[h, p, n] * dA + dt' * B[g, n] * x[h, p]            (fp32, in place)
//   y[h, p]        = sum_n state[h, p, n] * C[g, n] + D[h] * x[h, p]          g = h / (H / groups)
//
// Pure streaming: the fp32 state (H x P x N = 3.9 MB per sequence at 96 x 80 x 128) is read and written once, everything
// else is a few KB.  The reference gives a head to a 128-thread CTA whose four warps walk the head's P rows one after
// the other (96 CTAs, 20 dependent rows per warp).  Here a head is split over five 8-warp CTAs and a warp requests all
// the elements of its two rows before it uses the first (the whole state of a sequence in flight at once), while the
// per-head scalars (softplus, two exponentials) are computed once per CTA and the head's B / C values loaded once per
// warp, not once per row: with only four state elements per lane and row they would otherwise be most of the instructions.  A
// lane owns the same elements n = lane, lane + 32, ... of a row as in the reference and the row sum goes down the same
// shuffle tree, so state and y are bit-identical to the reference kernel's.
//
// The state rows are requested BEFORE the wait on the preceding kernel: the only writer of a state is this kernel one
// token earlier, never the kernel just before it in the stream (the conv step); x, dt, B and C are read after the wait.
#include "nmt_common.cuh"

namespace nmt {

constexpr int kSsmWarps = 8;

template <int NPER, int RPW>                                    // ceil(N / 32) state elements per lane and row; rows per warp
__global__ void __launch_bounds__(kSsmWarps * 32)
ssm_step_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt, const float* __restrict__ A_log,
                const __nv_bfloat16* __restrict__ B, const __nv_bfloat16* __restrict__ C, const float* __restrict__ D_param,
                const float* __restrict__ dt_bias, float* __restrict__ state, __nv_bfloat16* __restrict__ y,
                int H, int P, int N, int groups, float dt_min, float dt_max) {
    const int lane = threadIdx.x & 31;
    // A CTA owns kSsmWarps * RPW consecutive rows p of one (sequence, head); a warp RPW of them.  All of a warp's state
    // elements are requested before the first use; the per-head scalars are computed by one thread of the CTA, the
    // head's B / C values loaded once per warp.
    __shared__ float s_scalar[3];
    __shared__ int s_bc;
    const int bh = blockIdx.x;                                     // sequence * H + head
    const int p0 = (blockIdx.y * kSsmWarps + (threadIdx.x >> 5)) * RPW;
    float* s_base = state + ((int64_t)bh * P + min(p0, P - 1)) * N;
    float s[RPW][NPER];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
#pragma unroll
        for (int j = 0; j < NPER; ++j) {
            const int n = lane + 32 * j;
            s[r][j] = (p0 + r < P && n < N) ? s_base[r * N + n] : 0.f;
        }
    }
    pdl_wait();
    if (threadIdx.x == 0) {
        const int h = bh % H, b = bh / H;
        // softplus and the decay exactly as the reference writes them (ops/mamba2/ssm.cuh:72-79)
        float dt_v = __bfloat162float(dt[bh]);
        if (dt_bias) dt_v += dt_bias[h];
        const float sp = (dt_v > 20.f) ? dt_v : (dt_v < -20.f) ? 0.f : logf(1.f + expf(dt_v));
        dt_v = fminf(dt_max, fmaxf(dt_min, sp));
        s_scalar[0] = dt_v;
        s_scalar[1] = expf(-expf(A_log[h]) * dt_v);
        s_scalar[2] = D_param[h];
        s_bc = b * groups + h / (H / groups);                      // which [N] row of B and C this head reads
    }
    __syncthreads();
    if (p0 < P) {                                                  // warp-uniform
        const float dt_v = s_scalar[0], dA = s_scalar[1], Dh = s_scalar[2];
        const __nv_bfloat16* Bg = B + (int64_t)s_bc * N;
        const __nv_bfloat16* Cg = C + (int64_t)s_bc * N;
        float dtB[NPER], sC[NPER];
#pragma unroll
        for (int j = 0; j < NPER; ++j) {
            const int n = lane + 32 * j;
            dtB[j] = n < N ? __fmul_rn(dt_v, __bfloat162float(Bg[n])) : 0.f;
            sC[j] = n < N ? __bfloat162float(Cg[n]) : 0.f;
        }
        const __nv_bfloat16* x_head = x + (int64_t)bh * P;
        __nv_bfloat16* y_head = y + (int64_t)bh * P;
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            if (p0 + r >= P) break;                                // warp-uniform
            const float x_val = __bfloat162float(x_head[p0 + r]);
            float y_part = 0.f;
#pragma unroll
            for (int j = 0; j < NPER; ++j) {
                const int n = lane + 32 * j;
                if (n < N) {
                    // s * dA + (dt' * B) * x with the sum fused into the first product: the contraction the reference's
                    // kernel is compiled to, spelled out so that it does not depend on the compiler's choice here
                    const float s_new = __fmaf_rn(s[r][j], dA, __fmul_rn(dtB[j], x_val));
                    s_base[r * N + n] = s_new;
                    y_part = __fmaf_rn(s_new, sC[j], y_part);
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) y_part += __shfl_down_sync(0xffffffffu, y_part, off);
            if (lane == 0) y_head[p0 + r] = __float2bfloat16_rn(__fmaf_rn(Dh, x_val, y_part));
        }
    }
    pdl_trigger();
}

}  // namespace nmt

extern "C" {

int nmt_ssm_decode_step_bf16(const void* x, const void* dt, const float* A_log, const void* B, const void* C, const float* D,
                             const float* dt_bias, float* state, void* y, int64_t batch, int64_t heads, int64_t head_dim,
                             int64_t state_size, int64_t n_groups, float dt_min, float dt_max, void* stream) {
    using namespace nmt;
    if (batch < 0 || heads <= 0 || head_dim <= 0 || state_size <= 0 || n_groups <= 0 || (heads % n_groups) != 0) return NMT_ERR_SHAPE;
    if (state_size > 256 || heads > 0x7fffffff / head_dim) return NMT_ERR_UNSUPPORTED;
    if (batch == 0) return NMT_OK;
    if (!x || !dt || !A_log || !B || !C || !D || !state || !y) return NMT_ERR_NULL;
    auto odd = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 1u) != 0; };
    if (odd(x) || odd(dt) || odd(B) || odd(C) || odd(y) || !aligned4(A_log) || !aligned4(D) || !aligned4(state) ||
        (dt_bias && !aligned4(dt_bias)))
        return NMT_ERR_ALIGN;
    // Rows per warp: the first of 2, 4, 5, 1 whose CTA (8 warps) tiles a head's rows with the least waste.  Measured at the
    // model's 96 x 80 x 128: 3.8 us per launch with 2 or 4 rows per warp, 4.3 us with 1 or 5 (one sequence); 16.8 / 17.4 /
    // 17.6 / 23.4 us with 2 / 4 / 5 / 1 (eight sequences).
    int rpw = tune("ssm.rows_per_warp", 0);
    if (rpw != 1 && rpw != 2 && rpw != 4 && rpw != 5) {
        int64_t best_waste = -1;
        for (int cand : {2, 4, 5, 1}) {
            const int64_t per_cta = (int64_t)kSsmWarps * cand;
            const int64_t waste = (head_dim + per_cta - 1) / per_cta * per_cta - head_dim;
            if (best_waste < 0 || waste < best_waste) { best_waste = waste; rpw = cand; }
        }
    }
    const int64_t chunks = (head_dim + (int64_t)kSsmWarps * rpw - 1) / ((int64_t)kSsmWarps * rpw);
    if (batch * heads > 0x7fffffff || chunks > 65535 || batch * heads * head_dim > 0x7fffffff) return NMT_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto X = static_cast<const __nv_bfloat16*>(x);
    auto DT = static_cast<const __nv_bfloat16*>(dt);
    auto Bp = static_cast<const __nv_bfloat16*>(B);
    auto Cp = static_cast<const __nv_bfloat16*>(C);
    auto Y = static_cast<__nv_bfloat16*>(y);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(batch * heads), static_cast<unsigned>(chunks));
    cfg.blockDim = dim3(kSsmWarps * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
#define NMT_SSM_LAUNCH(NP, RW)                                                                                              \
    cudaLaunchKernelEx(&cfg, ssm_step_kernel<NP, RW>, X, DT, A_log, Bp, Cp, D, dt_bias, state, Y, static_cast<int>(heads),   \
                       static_cast<int>(head_dim), static_cast<int>(state_size), static_cast<int>(n_groups), dt_min, dt_max)
#define NMT_SSM_CASE(NP)                                                                                                    \
    do {                                                                                                                    \
        if (rpw == 5) NMT_SSM_LAUNCH(NP, 5); else if (rpw == 4) NMT_SSM_LAUNCH(NP, 4);                                      \
        else if (rpw == 2) NMT_SSM_LAUNCH(NP, 2); else NMT_SSM_LAUNCH(NP, 1);                                               \
    } while (0)
    const int nper = static_cast<int>((state_size + 31) / 32);
    if (nper <= 1) NMT_SSM_CASE(1);
    else if (nper <= 2) NMT_SSM_CASE(2);
    else if (nper <= 4) NMT_SSM_CASE(4);
    else NMT_SSM_CASE(8);
#undef NMT_SSM_CASE
#undef NMT_SSM_LAUNCH
    return finish_launch(1);
}

}  // extern "C"
