// A probe of the library's own safety net, for its tests: the bounded mbarrier wait that every TMA and tcgen05 kernel
// here relies on (mbarrier.cuh) is made to run out on purpose, in the only form that is harmless -- a barrier in
// shared memory that nothing will ever arrive at, no copy in flight, no tensor memory held, a limit of at most a
// tenth of a second -- so that a test can see the status bit, the abort flag that the block's other roles watch,
// and a context that goes on working afterwards.
#include "common.cuh"
#include "mbarrier.cuh"

namespace {

__global__ void wait_timeout_probe_kernel(long long limit, int* status, int* out) {
    __shared__ unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    bool ok = true;
    if (threadIdx.x == 0) ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, limit);   // nobody arrives
    __syncthreads();
    if (threadIdx.x == 0) out[0] = ok ? 1 : 0;          // what the waiting role was told
    if (threadIdx.x == 32) out[1] = abort_flag;         // what another role of the block sees
    // a second wait in the same block gives up at once, as the other roles' waits do after an abort
    if (threadIdx.x == 64) {
        const long long t0 = clock64();
        const bool again = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, limit);
        out[2] = again ? 1 : 0;
        out[3] = (clock64() - t0) < limit ? 1 : 0;
    }
}

}  // namespace

// limit_clocks: SM clocks the wait may take (a millisecond is about two million); out: int32[4] on the device:
// {the wait's answer, the abort flag as another warp sees it, a later wait's answer, whether that one returned early}.
VCB_API int vcb_selftest_wait_timeout(long long limit_clocks, int* status, int* out, cudaStream_t stream) {
    VCB_CHECK_ARG(limit_clocks > 0 && limit_clocks <= 200000000ll, "selftest_wait_timeout: a limit of %lld clocks (1 to 200,000,000)", limit_clocks);
    VCB_CHECK_ARG(status != nullptr && out != nullptr, "selftest_wait_timeout: status and out are required");
    wait_timeout_probe_kernel<<<1, 96, 0, stream>>>(limit_clocks, status, out);
    VCB_CHECK_LAUNCH("selftest_wait_timeout");
    return 0;
}
