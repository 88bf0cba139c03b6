// selftest.cu -- runs the give-up path of the library's bounded waits on purpose, safely.
//
// Every wait inside a kernel of this library has an iteration limit; when it runs out the kernel records an
// error word, returns, and the host reports MOTY_CUDA_EKERNEL.  That path never triggers in normal operation, so
// this file offers it on demand: three tiny kernels call the SAME wait functions as the production kernels
// (waits.cuh, gridbar.cuh) on something nobody will ever complete -- an mbarrier with no arrival pending, a grid
// barrier that expects one CTA more than the grid has -- with a limit of a few thousand polls (well under a
// millisecond).  Nothing faults, traps or hangs: each kernel polls, gives up, sets its error word and exits, and
// the context stays usable.  moty_cuda_kernel_status() must then report the failure, clear the words and put the
// barrier counters back, and the next ordinary call must work.
#include "kernels.cuh"
#include "gridbar.cuh"

namespace {

constexpr unsigned SELFTEST_LIMIT = 1u << 12;

__global__ void __launch_bounds__(64) selftest_mbar_kernel(int *err_word, int abortable) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const unsigned saddr = (unsigned)__cvta_generic_to_shared(&bar);
    if (threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr), "r"(1u));
        abort_flag = 0;
    }
    __syncthreads();
    // thread 0 waits for a phase that no arrival and no copy will ever complete; thread 32 (another "role") waits
    // on the same barrier and must leave as soon as the first raised the abort flag
    if (threadIdx.x == 0 || (abortable && threadIdx.x == 32)) {
        const bool ok = abortable ? moty_mbar_wait_abortable(saddr, 0, &abort_flag, threadIdx.x == 0 ? SELFTEST_LIMIT : 1u << 30)
                                  : moty_mbar_wait_bounded(saddr, 0, SELFTEST_LIMIT);
        if (!ok && threadIdx.x == 0) atomicExch(err_word, 1);
    }
}

__global__ void __launch_bounds__(32) selftest_gridbar_kernel(unsigned *bar, int *err_word) {
    __shared__ int gave_up;
    if (threadIdx.x == 0) gave_up = 0;
    __syncthreads();
    if (!grid_barrier_bounded(bar, &gave_up, gridDim.x + 1, SELFTEST_LIMIT))
        if (threadIdx.x == 0) atomicExch(err_word, 1);
}

}  // namespace

int launch_selftest_expire(int which, int *err_dev, unsigned *gridbar_words, cudaStream_t st) {
    if (which == 0) selftest_mbar_kernel<<<1, 64, 0, st>>>(err_dev + 0, 1);
    else if (which == 2) selftest_mbar_kernel<<<1, 64, 0, st>>>(err_dev + 2, 0);
    else if (which == 1) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2); cfg.blockDim = dim3(32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeCooperative;
        at[0].val.cooperative = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        CK(cudaLaunchKernelEx(&cfg, selftest_gridbar_kernel, gridbar_words, err_dev + 1));
        return 0;
    } else return moty_set_error(MOTY_CUDA_EARG, "selftest_expire_wait: which=%d (0 GEMM pipeline wait, 1 grid barrier, 2 bulk-copy wait)", which);
    CK(cudaGetLastError());
    return 0;
}
