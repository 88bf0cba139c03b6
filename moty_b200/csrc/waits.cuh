// waits.cuh -- the bounded mbarrier waits shared by every kernel that waits on an asynchronous copy or on a
// tensor-core commit.  Nothing in this library spins without a limit: a wait that runs out returns false, the
// kernel records that in the device error words (DevCtx::err_dev: [0] tensor-core GEMM, [1] grid barrier of the
// one-launch MoE/FFN decode kernels, [2] Q4R4/Q8R4 decode kernels fed by bulk copies), finishes without the data
// and the host reports MOTY_CUDA_EKERNEL (the host-pointer entries on return, device-resident callers through
// moty_cuda_kernel_status).  The limits are parameters so that the give-up path can be exercised with a short
// one (selftest.cu) by the very functions the production kernels call.
#pragma once
#include <stdint.h>

__device__ __forceinline__ bool moty_mbar_try(unsigned bar_saddr, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar_saddr), "r"(parity) : "memory");
    return ok != 0;
}

// plain bounded wait: false when `limit` polls saw the phase unfinished
__device__ __forceinline__ bool moty_mbar_wait_bounded(unsigned bar_saddr, unsigned parity, unsigned limit) {
    for (unsigned it = 0; it < limit; it++)
        if (moty_mbar_try(bar_saddr, parity)) return true;
    return false;
}

// bounded wait of a kernel with several roles (producer / issuer / epilogue): returns false when the limit is hit
// (and raises the CTA's abort flag) or when another role raised it, so that all roles leave together
__device__ __forceinline__ bool moty_mbar_wait_abortable(unsigned bar_saddr, unsigned parity, volatile int *abort_flag,
                                                         unsigned limit) {
    for (unsigned it = 0; it < limit; it++) {
        if (moty_mbar_try(bar_saddr, parity)) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
