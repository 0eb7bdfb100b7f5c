// mbarrier + TMA bulk-copy (cp.async.bulk, 1-D, no tensor map) helpers for the staged kernels.
//
// Rows of every tensor on this path are contiguous and a multiple of 16 bytes, so a tile of consecutive
// rows is ONE contiguous 16-byte-aligned range: the untiled bulk copy moves it with a single instruction
// and completes on an mbarrier in shared memory.  All copies are CTA-local, unicast, from this GPU's memory.
//
// Every wait is bounded: after kSpinLimit polls a waiter records the timeout in a device counter and the
// kernel winds down instead of spinning forever (the host reads the counter with nmt_device_wait_timeouts()).
#pragma once

#include "nmt_common.cuh"

namespace nmt {

constexpr uint32_t kSpinLimit = 1u << 21;      // polls of ~2 us each: a few seconds at most
constexpr uint32_t kSuspendHintNs = 2000;

static __device__ unsigned int g_wait_timeouts = 0;     // one counter per translation unit

void register_timeout_reader(cudaError_t (*reader)(unsigned int*));   // runtime.cu
#define NMT_DEFINE_TIMEOUT_READER()                                                              \
    static cudaError_t nmt_read_timeouts(unsigned int* v) {                                      \
        return cudaMemcpyFromSymbol(v, g_wait_timeouts, sizeof(unsigned int));                   \
    }                                                                                            \
    static const int nmt_timeout_reader_registered = (register_timeout_reader(nmt_read_timeouts), 0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs) : "memory");
    return ok != 0;
}
// Returns false (and counts a timeout) if the phase did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait_limited(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    atomicAdd(&g_wait_timeouts, 1u);
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return mbar_wait_limited(bar, parity, kSpinLimit); }
// The same wait as a plain poll (mbarrier.test_wait returns at once, no suspension): for waiters that expect the phase
// to complete within a microsecond or so and must not lose that long to a suspended thread's wake-up.  Bounded too.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_poll(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < (1u << 26); ++i)          // ~50 ns per poll: a few seconds at most
        if (mbar_test_wait(bar, parity)) return true;
    atomicAdd(&g_wait_timeouts, 1u);
    return false;
}

// global -> shared bulk copy; completion (byte count) is signalled on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk async-group.
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
// Makes generic-proxy writes to shared memory visible to the async proxy (before a bulk store reads them).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}
__device__ __forceinline__ void sts128(void* p, const uint4& v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(smem_u32(p)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

constexpr int kMaxDynSmem = 227 * 1024;

}  // namespace nmt
