// gridbar.cuh -- a counting barrier over all CTAs of a cooperative launch, with a BOUNDED wait.
//
// bar[0] counts arrivals, bar[1] is the generation.  The last CTA to arrive re-zeroes the count
// (ready for the next launch) and bumps the generation with release semantics; the others poll the
// generation with acquire loads.  Every CTA must be resident (cooperative launch) or the wait
// cannot complete; if it does not complete within the limit anyway, the caller is told so, sets
// an error word and leaves: nothing spins for ever.
#pragma once
#include "common.cuh"

constexpr unsigned GRIDBAR_SPIN_LIMIT = 4u << 20;      // polls of ~0.3-1 us each: around a second

__device__ __forceinline__ unsigned gb_ld_acquire(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned gb_add_acq_rel(unsigned *p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void gb_add_release(unsigned *p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ALL threads of the CTA.  Returns false when the wait expired (to every thread).
// Global writes made by any thread of any CTA before the barrier are visible to every thread after it.
// `expected` arrivals complete the barrier (the grid size in every production kernel) and `limit` polls bound the
// wait; both are parameters so that the give-up path can be run on purpose with a count nobody completes.
__device__ __forceinline__ bool grid_barrier_bounded(unsigned *bar, int *gave_up_smem, unsigned expected = 0,
                                                     unsigned limit = GRIDBAR_SPIN_LIMIT) {
    if (expected == 0) expected = gridDim.x;
    __syncthreads();                                   // this CTA's writes are done (and ordered before thread 0's release)
    if (threadIdx.x == 0) {
        const unsigned gen = gb_ld_acquire(bar + 1);   // cannot change before this CTA has arrived
        const unsigned old = gb_add_acq_rel(bar, 1u);
        if (old == expected - 1) {
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(bar), "r"(0u) : "memory");
            gb_add_release(bar + 1, 1u);
        } else {
            unsigned n = 0;
            while (gb_ld_acquire(bar + 1) == gen) {
                if (++n > limit) { *gave_up_smem = 1; break; }
            }
        }
    }
    __syncthreads();
    return *gave_up_smem == 0;
}
