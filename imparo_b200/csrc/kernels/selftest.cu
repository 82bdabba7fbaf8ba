// Self-tests of the failure paths that ordinary runs never take.
//
// Every device wait of this engine is bounded: a wait that runs out makes its kernel record
// IMPARO_ST_WAIT_LIMIT in the status word and return, so that the context stays usable and the
// host learns of it at its next status read.  The kernel below waits on an mbarrier that nothing
// ever completes, with a small poll limit, so that this path can be exercised without hanging or
// faulting anything.
#include "tcgen05.cuh"

namespace imparo {

__global__ void wait_runs_out_kernel(int* status, uint32_t limit, int* outcome) {
    __shared__ __align__(8) uint64_t bar;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool done = tc::mbar_wait(&bar, 0, limit);         // nobody arrives: parity 0 never completes
        if (!done) report(status, IMPARO_ST_WAIT_LIMIT, 90, (int)limit, 0);
        *outcome = done ? 1 : 2;                                  // the kernel went on to its end either way
    }
}

}  // namespace imparo

// limit: polls before the wait gives up (at most 100000 here: a fraction of a second).
extern "C" int imparo_selftest_wait_limit(int* status, int limit, int* outcome, cudaStream_t stream) {
    if (limit < 1 || limit > 100000) return -2;
    launch(imparo::wait_runs_out_kernel, dim3(1), dim3(32), 0, stream, status, (uint32_t)limit, outcome);
    IMPARO_CHECK_LAUNCH();
    return 0;
}
