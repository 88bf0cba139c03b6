// router.cu -- MoE router (softmax + greedy top-K) and the greedy-token argmax.
#include "kernels.cuh"
#include "route.cuh"

// One warp per token row; the arithmetic is route_row_warp (route.cuh).
__global__ void __launch_bounds__(128) route_kernel(const float *__restrict__ logits, int rows, int E, int K,
                                                    int *__restrict__ idx, float *__restrict__ w,
                                                    float *__restrict__ probs, int do_softmax, int norm_topk,
                                                    const float *__restrict__ bias) {
    extern __shared__ __align__(16) float sm[];            // four scratch rows of E floats (2 E for the sigmoid gate), 16-byte aligned
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + warp;
    pdl_trigger();
    pdl_wait();                              // the logits come from the kernel before this one
    if (row >= rows) return;
    if (do_softmax == 2) {                   // sigmoid + expert bias (LFM2)
        route_row_warp_sigmoid(logits + (size_t)row * E, bias, E, K, sm + (size_t)warp * 2 * ((E + 3) & ~3), lane,
                               idx + (size_t)row * K, w + (size_t)row * K);
        return;
    }
    route_row_warp(logits + (size_t)row * E, E, K, sm + (size_t)warp * ((E + 3) & ~3), do_softmax, norm_topk, lane,
                   idx + (size_t)row * K, w + (size_t)row * K, probs ? probs + (size_t)row * E : nullptr);
}

// do_softmax: 0 = top-K of given probabilities, 1 = softmax then top-K, 2 = sigmoid + bias gate (bias may be null)
int launch_route(const float *logits, int rows, int E, int K, int *idx, float *w, float *probs,
                 int do_softmax, int norm_topk, cudaStream_t st, const float *bias) {
    if (rows <= 0) return 0;
    if (E <= 0 || E > 4096 || K <= 0 || K > 64 || K > E)
        return moty_set_error(MOTY_CUDA_EARG, "route: E=%d K=%d (E <= 4096, K <= 64, K <= E)", E, K);
    size_t smem = (size_t)4 * ((E + 3) & ~3) * sizeof(float) * (do_softmax == 2 ? 2 : 1);
    if (smem > 48 * 1024) CK(cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(moty_launch_pdl(route_kernel, dim3((rows + 3) / 4), dim3(128), smem, st, logits, rows, E, K, idx, w, probs,
                       do_softmax, norm_topk, bias));
    return 0;
}

// ---------------------------------------------------------------------------
// moty_argmax_v (nn/sample.c:9-13): first index of the maximum.  Two passes:
// per-CTA partials (value, lowest index), then one CTA combines them.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void argmax_combine(float &bv, int &bi, float ov, int oi) {
    if (oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
}

__global__ void __launch_bounds__(256) argmax_part_kernel(const float *__restrict__ v, int n, float *pv, int *pi) {
    __shared__ float sv[8]; __shared__ int si[8];
    float bv = 0.f; int bi = -1;
    pdl_trigger();
    pdl_wait();
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) {
        float x = v[i];
        if (bi < 0 || x > bv) { bv = x; bi = i; }       // ascending i per thread: strict > keeps the first
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, d); int oi = __shfl_xor_sync(0xffffffffu, bi, d);
        argmax_combine(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < 8; k++) argmax_combine(bv, bi, sv[k], si[k]);
        pv[blockIdx.x] = bv; pi[blockIdx.x] = bi;
    }
}

__global__ void __launch_bounds__(256) argmax_final_kernel(const float *pv, const int *pi, int nparts, int *out) {
    __shared__ float sv[8]; __shared__ int si[8];
    float bv = 0.f; int bi = -1;
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < nparts; i += 256) argmax_combine(bv, bi, pv[i], pi[i]);
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, d); int oi = __shfl_xor_sync(0xffffffffu, bi, d);
        argmax_combine(bv, bi, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < 8; k++) argmax_combine(bv, bi, sv[k], si[k]);
        *out = bi < 0 ? 0 : bi;
    }
}

// scratch: 256 partial (value, index) pairs, provided by the caller
int launch_argmax_scratch(const float *v, int n, int *out, float *pv, int *pi, cudaStream_t st) {
    if (n <= 0) return moty_set_error(MOTY_CUDA_EARG, "argmax: n=%d", n);
    int parts = (n + 255) / 256; if (parts > 256) parts = 256;
    CK(moty_launch_pdl(argmax_part_kernel, dim3(parts), dim3(256), (size_t)0, st, v, n, pv, pi));
    CK(moty_launch_pdl(argmax_final_kernel, dim3(1), dim3(256), (size_t)0, st, (const float *)pv, (const int *)pi, parts, out));
    return 0;
}
