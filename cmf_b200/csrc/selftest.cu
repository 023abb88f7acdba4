// Self-test of the bounded-wait path every kernel of this library relies on: a kernel waits on an
// mbarrier that nobody ever arrives on, with a small poll budget, gives up, records the site and
// returns through its normal exit; the host then reports CMFC_ERR_DEVICE_WAIT and the context stays
// usable.  Not reachable from any product entry; it exists so that the failure path can be
// exercised without hanging or faulting a GPU.
#include "../../include/cmf_cuda.h"
#include "runtime.h"

using namespace cmfc;

namespace {

constexpr uint32_t SELFTEST_SITE = 9;

__global__ void __launch_bounds__(64) wait_runs_out_kernel(uint32_t* status, uint32_t polls) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    // warp 0 waits for a phase that never completes; warp 1 waits too and leaves early once warp 0
    // has flagged the abort (the way the other roles of a real kernel unwind)
    if (threadIdx.x == 0) mbar_wait_budget(&bar, 0u, &abort_flag, SELFTEST_SITE, polls);
    if (threadIdx.x == 32) mbar_wait_budget<100>(&bar, 0u, &abort_flag, SELFTEST_SITE + 1, 64u * polls);
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicCAS(status, 0u, 0x700u | abort_flag);
}

}  // namespace

extern "C" int cmfc_selftest_wait_timeout(uint32_t polls) {
    if (polls == 0 || polls > (1u << 16)) return fail(ERR_BAD_ARG, "selftest_wait_timeout: polls must be in [1, 65536]");
    Context* c = ctx();
    if (!c) return last_error().empty() ? fail(ERR_CUDA, "no CUDA device") : ERR_CUDA;
    wait_runs_out_kernel<<<1, 64, 0, c->stream>>>(c->status, polls);
    c->launches++;
    CMFC_CUDA(cudaGetLastError());
    return check_status(c, "selftest_wait_timeout");
}
