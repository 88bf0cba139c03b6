// hostio.cu -- moving a call's activations and results between the caller's PINNED host buffers and the device with
// kernels instead of copy-engine transfers, for the host-pointer entries (moty_cuda_mat_apply): a copy-engine transfer
// of a few KB costs 4-5 us of latency at each end of a product that itself takes 5-10 us, and the stream
// synchronisation after it a few more.  Page-locked host memory is mapped into the device's address space, so
//   stage_in_kernel   reads x from the host buffer (coalesced 16-byte loads over PCIe) into the device scratch,
//   tail_out_kernel   writes y from the device scratch to the host buffer (coalesced 16-byte stores), fences, and the
//                     last CTA to finish stores the call's sequence number (counted on the device) to a pinned flag word,
// and the host waits for that word (bounded; then it falls back to a stream synchronisation) instead of synchronising.
// Both are chained to the product between them by programmatic dependent launch, and a call that repeats (same matrix,
// same buffers: a decode loop) is replayed as one CUDA graph of the three launches (api.cu), one submission instead of three.  Pageable buffers (malloc) are not
// mapped: those calls keep the copy-engine path.
#include "kernels.cuh"

namespace {

__global__ void __launch_bounds__(256) stage_in_kernel(float *dst, const float *src_host, long long n) {
    pdl_trigger();
    pdl_wait();                                            // the scratch may still be read by the launch before
    const long long n4 = n / 4, i0 = (long long)blockIdx.x * 256 + threadIdx.x, step = (long long)gridDim.x * 256;
    for (long long i = i0; i < n4; i += step) reinterpret_cast<float4 *>(dst)[i] = reinterpret_cast<const float4 *>(src_host)[i];
    for (long long i = n4 * 4 + i0; i < n; i += step) dst[i] = src_host[i];
}

// ctr[0]: CTAs that have finished (zero between launches); ctr[1]: calls completed so far -- the value the flag word gets,
// kept on the device so that a replayed CUDA graph of a call needs no new argument
__global__ void __launch_bounds__(256) tail_out_kernel(float *dst_host, const float *src, long long n, unsigned *ctr,
                                                       volatile unsigned *flag_host) {
    __shared__ bool last;
    pdl_trigger();
    pdl_wait();                                            // the product's results
    const long long n4 = n / 4, i0 = (long long)blockIdx.x * 256 + threadIdx.x, step = (long long)gridDim.x * 256;
    for (long long i = i0; i < n4; i += step) reinterpret_cast<float4 *>(dst_host)[i] = reinterpret_cast<const float4 *>(src)[i];
    for (long long i = n4 * 4 + i0; i < n; i += step) dst_host[i] = src[i];
    __threadfence_system();                                // this thread's stores to the host are ordered before the count
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(ctr, 1u) == gridDim.x - 1;
    __syncthreads();
    if (last && threadIdx.x == 0) {
        ctr[0] = 0;                                        // zero between launches
        const unsigned seq = ctr[1] + 1;
        ctr[1] = seq;
        __threadfence_system();
        *flag_host = seq;
    }
}

}  // namespace

int launch_stage_in(float *dst, const float *src_host, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    long long ctas = (n / 4 + 255) / 256;
    if (ctas < 1) ctas = 1;
    if (ctas > 16) ctas = 16;
    CK(moty_launch_pdl(stage_in_kernel, dim3((unsigned)ctas), dim3(256), (size_t)0, st, dst, src_host, n));
    return 0;
}

int launch_tail_out(float *dst_host, const float *src, long long n, unsigned *ctr, unsigned *flag_host, int sms, cudaStream_t st) {
    long long ctas = (n / 4 + 1023) / 1024;                // four 16-byte stores per thread
    if (ctas < 1) ctas = 1;
    if (ctas > sms) ctas = sms;
    CK(moty_launch_pdl(tail_out_kernel, dim3((unsigned)ctas), dim3(256), (size_t)0, st, dst_host, src, n, ctr,
                       (volatile unsigned *)flag_host));
    return 0;
}
