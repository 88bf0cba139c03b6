// resnorm.cuh -- the residual step and RMS norm in front of a one-token product, formed by every CTA of that product
// for itself (256 threads), so that a decode layer needs no launch of its own for them:
//     v   = x + t                         (hw/hw_ops.h:30-32; engines/qwen.c:699,711)         when g_t == nullptr
//     v   = x + (t * r_t) * g_t           (engines/gemma.c:470-474, 480-482: the post-block norm, then the add)
//     row = (v * r_v) * g_x               (hw/hw_ops.h:14-18 / gnorm_row, engines/gemma.c:279-284)
// with r = 1 / sqrtf((float)(mean of squares in double) + eps).  Element for element and sum for sum the order of the
// separate launches (rmsnorm_rows_kernel<true>, normadd_rmsnorm_rows_kernel in norm.cu: thread i takes elements
// i, i + 256, ... in ascending order, the same shuffle tree, the eight warp sums added in order), so both routes give
// the same bits.  The row is left in xf[I] (shared memory), the sum v goes to xout from the CTA that `writer` names
// (to another buffer than x: the other CTAs are still reading x), and the function returns the CTA-wide max |row|.
// I <= 4096.  Every thread of the CTA must call it; red64 is 8 doubles, red32 8 floats of shared memory.
#pragma once
#include "common.cuh"

__device__ __forceinline__ double resnorm_block_sum(double v, double *red64, bool again) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (again) __syncthreads();                               // red64 may still be read from the sum before this one
    if ((threadIdx.x & 31) == 0) red64[threadIdx.x >> 5] = v;
    __syncthreads();
    double s = 0;
    for (int i = 0; i < 8; i++) s += red64[i];
    return s;
}

__device__ __forceinline__ float resnorm_row(const float *x, const float *t, const float *g_t, const float *g_x, float *xout,
                                             float eps, int I, float *xf, double *red64, float *red32, bool writer) {
    float rt = 0.f;
    if (g_t) {                                                // the norm of t first: one more pass over t (it sits in L2)
        double ms = 0;
        for (int i = threadIdx.x; i < I; i += 256) { const float a = t[i]; ms += (double)a * (double)a; }
        ms = resnorm_block_sum(ms, red64, false);
        rt = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / I), eps)));
    }
    // loads go out four rounds at a time (a row of 1024 is one round trip), the gains of the first four with them
    double ms = 0;
    float gv[4];
#pragma unroll
    for (int j = 0; j < 4; j++) { const int i = threadIdx.x + 256 * j; gv[j] = i < I ? g_x[i] : 0.f; }
    for (int i0 = threadIdx.x; i0 < I; i0 += 1024) {
        float xv[4], tv[4], g1[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = i0 + 256 * j;
            xv[j] = i < I ? x[i] : 0.f; tv[j] = i < I ? t[i] : 0.f; g1[j] = (g_t && i < I) ? g_t[i] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = i0 + 256 * j;
            if (i < I) {
                const float v = g_t ? __fadd_rn(xv[j], __fmul_rn(__fmul_rn(tv[j], rt), g1[j])) : __fadd_rn(xv[j], tv[j]);
                xf[i] = v;
                if (writer) xout[i] = v;
                ms += (double)v * (double)v;
            }
        }
    }
    ms = resnorm_block_sum(ms, red64, g_t != nullptr);
    const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / I), eps)));
    float amax = 0.f;
    for (int i0 = threadIdx.x; i0 < I; i0 += 1024) {
        if (i0 >= 1024) {
#pragma unroll
            for (int j = 0; j < 4; j++) { const int i = i0 + 256 * j; gv[j] = i < I ? g_x[i] : 0.f; }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i = i0 + 256 * j;
            if (i < I) {
                const float nv = __fmul_rn(__fmul_rn(xf[i], r), gv[j]);
                xf[i] = nv;
                amax = fmaxf(amax, fabsf(nv));
            }
        }
    }
    amax = warp_max_f32(amax);
    if ((threadIdx.x & 31) == 0) red32[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red32[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red32[i]);
    return amax;
}
