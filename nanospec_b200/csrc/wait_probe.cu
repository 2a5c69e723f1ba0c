// A bounded wait that runs out, on purpose and safely: the error path that the tcgen05 and TMA kernels
// take when an mbarrier never completes (mbar_wait gives up, the kernel records a code in the error word
// and returns) shown on its own.  One block, no cluster, no copy and no tensor-core operation in flight:
// one thread waits on a barrier at which nobody ever arrives, with the limit given by the caller, gives
// up, records the code and the kernel ends normally.  The production kernels are never starved to get there.
#include "tcgen05_utils.cuh"

namespace {

constexpr int kWaitProbeCode = 31;

__global__ void __launch_bounds__(32) wait_probe_kernel(int* error_flag, unsigned long long limit_ns, int* waited_ok) {
    __shared__ __align__(8) unsigned long long bar;
    ns_pdl_launch_dependents();
    ns_pdl_wait();
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const bool ok = mbar_wait(smem_u32(&bar), 0, limit_ns, 0u);  // phase 0 never completes: nobody arrives; the clock is read at every poll
        if (!ok) atomicExch(error_flag, kWaitProbeCode);
        *waited_ok = ok ? 1 : 0;
    }
}

}  // namespace

// `limit_ns`: how long the one thread waits before it gives up (at most one second is accepted).
// `error_flag`: the word that the other kernels' waits report to; `waited_ok`: 1 if the wait completed (it cannot), else 0.
NS_API int ns_wait_probe(int* error_flag, long long limit_ns, int* waited_ok, cudaStream_t stream) {
    if (!error_flag || !waited_ok) NS_FAIL(NS_ERR_ARGUMENT, "ns_wait_probe: null pointer");
    if (limit_ns < 1000 || limit_ns > 1000000000ll)
        NS_FAIL(NS_ERR_ARGUMENT, "ns_wait_probe: limit of %lld ns (1 us to 1 s)", limit_ns);
    NS_LAUNCH(wait_probe_kernel, 1, 32, 0, stream, error_flag, (unsigned long long)limit_ns, waited_ok);
    NS_CHECK_LAUNCH("ns_wait_probe");
    return NS_OK;
}
