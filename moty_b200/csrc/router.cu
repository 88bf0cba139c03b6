// router.cu -- MoE router (softmax + greedy top-K) and the greedy-token argmax.
#include "kernels.cuh"

// One warp per token row.
//
// Softmax follows moty_hw_softmax_ref (hw/hw_ops.h:22-26): running maximum from
// -1e30, e = exp(x - m) rounded to f32, the sum taken SEQUENTIALLY in index
// order in f32 (one lane does it: E is at most a few thousand), then one true
// division per element.  exp is evaluated in f64 and rounded once, which agrees
// with a correctly rounded expf; a libm expf may differ from that by one ulp on
// roughly one value in a thousand, which does not move the ranking in practice.
//
// Top-K follows moty_moe_topk (runtime/moecache.c:97-111): K rounds of "largest
// value not yet taken", strict > against a floor of -1e30, so equal values go to
// the lowest index.  The argmax with lowest-index tie-break is order independent,
// so the lanes can scan disjoint slices and combine.
__global__ void __launch_bounds__(128) route_kernel(const float *__restrict__ logits, int rows, int E, int K,
                                                    int *__restrict__ idx, float *__restrict__ w,
                                                    float *__restrict__ probs, int do_softmax, int norm_topk) {
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) return;
    float *p = sm + (size_t)warp * E;
    const float *lg = logits + (size_t)row * E;
    for (int e = lane; e < E; e += 32) p[e] = lg[e];
    __syncwarp();
    if (do_softmax) {
        float m = -1e30f;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, p[e]);
        m = warp_max_f32(m);
        for (int e = lane; e < E; e += 32) p[e] = (float)exp((double)__fsub_rn(p[e], m));
        __syncwarp();
        float total = 0.f;
        if (lane == 0)
            for (int e = 0; e < E; e++) total = __fadd_rn(total, p[e]);
        total = __shfl_sync(0xffffffffu, total, 0);
        for (int e = lane; e < E; e += 32) p[e] = __fdiv_rn(p[e], total);
        __syncwarp();
        if (probs)
            for (int e = lane; e < E; e += 32) probs[(size_t)row * E + e] = p[e];
    }
    // K rounds; a taken entry is remembered in a per-lane bitmask over its own slice
    // (E <= 4096 -> at most 128 entries per lane -> 4 words)
    unsigned taken[4] = {0u, 0u, 0u, 0u};
    float wsum = 0.f;
    float mine = 0.f;                        // lane k keeps weight k (K <= 64: two per lane)
    float mine2 = 0.f;
    for (int k = 0; k < K; k++) {
        float bv = -1e30f; int bi = -1;
        for (int e = lane, j = 0; e < E; e += 32, j++) {
            if (taken[j >> 5] & (1u << (j & 31))) continue;
            float v = p[e];
            if (v > bv) { bv = v; bi = e; }
        }
        // combine: larger value wins, equal values -> lower index; -1 (nothing) loses
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, d);
            int oi = __shfl_xor_sync(0xffffffffu, bi, d);
            bool take = (oi >= 0) && (bi < 0 || ov > bv || (ov == bv && oi < bi));
            if (take) { bv = ov; bi = oi; }
        }
        if (bi >= 0 && (bi & 31) == lane) { int j = bi >> 5; taken[j >> 5] |= 1u << (j & 31); }
        if (lane == 0) idx[(size_t)row * K + k] = bi;
        if ((k & 31) == lane) { if (k < 32) mine = bv; else mine2 = bv; }
        wsum = __fadd_rn(wsum, bv);          // sequential sum in selection order
    }
    if (norm_topk && wsum > 0.f) { mine = __fdiv_rn(mine, wsum); mine2 = __fdiv_rn(mine2, wsum); }
    if (lane < K) w[(size_t)row * K + lane] = mine;
    if (lane + 32 < K) w[(size_t)row * K + lane + 32] = mine2;
}

int launch_route(const float *logits, int rows, int E, int K, int *idx, float *w, float *probs,
                 int do_softmax, int norm_topk, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (E <= 0 || E > 4096 || K <= 0 || K > 64 || K > E)
        return moty_set_error(MOTY_CUDA_EARG, "route: E=%d K=%d (E <= 4096, K <= 64, K <= E)", E, K);
    size_t smem = (size_t)4 * E * sizeof(float);
    if (smem > 48 * 1024) CK(cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    route_kernel<<<(rows + 3) / 4, 128, smem, st>>>(logits, rows, E, K, idx, w, probs, do_softmax, norm_topk);
    CK(cudaGetLastError());
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
    argmax_part_kernel<<<parts, 256, 0, st>>>(v, n, pv, pi);
    CK(cudaGetLastError());
    argmax_final_kernel<<<1, 256, 0, st>>>(pv, pi, parts, out);
    CK(cudaGetLastError());
    return 0;
}
