// Self-test of the bounded wait that every staged (bulk-copy) kernel of this library relies on.
//
// A wait that can never be satisfied is made on purpose, in the harmless form: one thread of one tiny CTA arms an
// mbarrier in its own shared memory for bytes that no copy will ever deliver and waits for it with a limit of a few
// polls.  The wait runs out after microseconds, is counted exactly like a run-out wait in a product kernel
// (mbar_wait_limited is the function behind every mbar_wait), the kernel returns normally and the context stays
// usable.  Nothing faults, traps or spins.
#include "nmt_tma.cuh"

namespace nmt {

NMT_DEFINE_TIMEOUT_READER();

__global__ void __launch_bounds__(32)
wait_runs_out_kernel(uint32_t polls, int* gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
        mbar_arrive_expect_tx(&bar, 16);                  // 16 bytes that nothing is going to copy
        const bool done = mbar_wait_limited(&bar, 0, polls);
        if (gave_up) *gave_up = done ? 0 : 1;
    }
}

}  // namespace nmt

extern "C" int nmt_selftest_wait_runs_out(int polls, int* gave_up_device, void* stream) {
    if (polls < 1 || polls > 4096) return NMT_ERR_SHAPE;
    nmt::wait_runs_out_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint32_t>(polls), gave_up_device);
    return nmt::finish_launch(1);
}
