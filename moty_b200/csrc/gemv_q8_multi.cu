// gemv_q8_multi.cu -- several independent Q8_0 decode products in ONE launch.
//
// A decode step is full of small matrices whose own GEMV launch costs more than their bytes: a 1-3 MB matrix is
// 0.2-0.5 us of HBM time behind 4-5 us of launch, prologue and tail.  This kernel takes up to eight (matrix, row)
// pairs -- moty_matmul_q_s with S = 1 for each (nn/matmul.c:51-66, IDOT=1), e.g. the q, k and v projections of a
// layer, or independent products of a benchmark pass -- cuts ALL their rows into units of two rows and deals the
// units round-robin to one persistent grid, so the fixed cost is paid once and the tail is one unit long.
// Every CTA quantizes each activation row (moty_hw_qrow_i8, hw/hw_quant.h:9-16: exact amax, true division,
// round-half-even) into shared memory behind its first weight loads.
// Same dp4a arithmetic and the same (scale[o] * sx) * (float)dot epilogue as q8_stream_kernel: same bits.
// Limits: I a multiple of 16, I <= 4096 (longer rows need the K split of the single-matrix kernel), x 16-byte aligned.
#include "kernels.cuh"
#include <string.h>

namespace {

constexpr int MULTI_MAX = 8, MR = 2, MLPR = 8;

struct MultiArgs {
    const int8_t *w[MULTI_MAX]; const float *scale[MULTI_MAX]; const float *x[MULTI_MAX]; float *y[MULTI_MAX];
    int O[MULTI_MAX], I16[MULTI_MAX], xoff[MULTI_MAX];     // xoff: where matrix m's codes start in shared memory (bytes)
    int ustart[MULTI_MAX + 1];                             // prefix of units (row pairs) per matrix
    int n;
};

__global__ void __launch_bounds__(256, 2) q8_multi_kernel(MultiArgs a) {
    extern __shared__ int4 smem4[];
    __shared__ float red[8];
    __shared__ float sx_s[MULTI_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nunits = a.ustart[a.n], nwarps = gridDim.x * 8;
    int8_t *xq_s = reinterpret_cast<int8_t *>(smem4);

    int4 wv[MR][MLPR];
    float sc[MR];
    int um = 0, ur = 0;                                    // matrix and first row of the unit in flight
    auto issue = [&](int u) {
        int m = 0;
        while (m + 1 < a.n && u >= a.ustart[m + 1]) m++;
        um = m; ur = (u - a.ustart[m]) * MR;
        const int I16 = a.I16[m], O = a.O[m];
#pragma unroll
        for (int r = 0; r < MR; r++) {
            const int o = ur + r < O ? ur + r : O - 1;
            const int4 *p = reinterpret_cast<const int4 *>(a.w[m]) + (size_t)o * I16;
#pragma unroll
            for (int j = 0; j < MLPR; j++) {
                const int k = j * 32 + lane;
                wv[r][j] = k < I16 ? ldg_stream16(p + k) : make_int4(0, 0, 0, 0);
            }
            sc[r] = __ldg(a.scale[m] + o);
        }
    };
    int u = blockIdx.x * 8 + warp;
    pdl_trigger();
    if (u < nunits) issue(u);                              // weights only: may run before the previous kernel has finished
    pdl_wait();                                            // activations and outputs from here on

    for (int m = 0; m < a.n; m++) {                        // quantize every row: two passes over x (it sits in L2)
        const int I4 = a.I16[m] * 4;
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x[m]);
        float amax = 0.f;
        for (int i = threadIdx.x; i < I4; i += 256) {
            const float4 v = x4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        amax = warp_max_f32(amax);
        __syncthreads();                                   // red[] of the previous matrix has been read
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
        const float sx = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, sx);
        int *xq = reinterpret_cast<int *>(xq_s + a.xoff[m]);
        for (int i = threadIdx.x; i < I4; i += 256) {
            const float4 v = x4[i];
            const int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
            const int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
            xq[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        if (threadIdx.x == 0) sx_s[m] = sx;
    }
    __syncthreads();

    while (u < nunits) {
        const int m = um, r0 = ur, I16 = a.I16[m], O = a.O[m];
        const int4 *xs = reinterpret_cast<const int4 *>(xq_s + a.xoff[m]);
        int dot[MR];
#pragma unroll
        for (int r = 0; r < MR; r++) dot[r] = 0;
#pragma unroll
        for (int j = 0; j < MLPR; j++) {
            if (j * 32 < I16) {                            // warp-uniform
                int k = j * 32 + lane; k = k < I16 ? k : I16 - 1;      // weights past the row were loaded as zeros
                const int4 xv = xs[k];
#pragma unroll
                for (int r = 0; r < MR; r++) dot[r] = dp4a4(wv[r][j], xv, dot[r]);
            }
        }
        const float s0 = sc[0], s1 = sc[1], sx = sx_s[m];
        u += nwarps;
        if (u < nunits) issue(u);                          // the next unit's loads go out before this result is written
#pragma unroll
        for (int r = 0; r < MR; r++) dot[r] = warp_sum_i32(dot[r]);
        if (lane < MR && r0 + lane < O) {
            // (scale[o] * sx) * (float)dot, left to right (nn/matmul.c:34)
            const int d = lane == 0 ? dot[0] : dot[1];
            a.y[m][r0 + lane] = __fmul_rn(__fmul_rn(lane == 0 ? s0 : s1, sx), (float)d);
        }
    }
}

}  // namespace

bool q8_multi_supported(int I) { return I % 16 == 0 && I >= 16 && I <= 4096; }

int launch_q8_multi(int n, const int8_t *const *w, const float *const *scale, const float *const *x, float *const *y,
                    const int *O, const int *I, int sms, cudaStream_t st) {
    if (n < 1 || n > MULTI_MAX) return moty_set_error(MOTY_CUDA_EARG, "q8_multi: %d matrices (1..%d)", n, MULTI_MAX);
    MultiArgs a;
    memset(&a, 0, sizeof a);
    a.n = n;
    int units = 0, xoff = 0;
    for (int m = 0; m < n; m++) {
        if (!q8_multi_supported(I[m]) || O[m] < 1 || (reinterpret_cast<uintptr_t>(x[m]) & 15))
            return moty_set_error(MOTY_CUDA_EARG, "q8_multi: matrix %d is %dx%d (rows of 16..4096 bytes, x 16-byte aligned)", m, O[m], I[m]);
        a.w[m] = w[m]; a.scale[m] = scale[m]; a.x[m] = x[m]; a.y[m] = y[m]; a.O[m] = O[m]; a.I16[m] = I[m] / 16;
        a.xoff[m] = xoff; xoff += I[m];
        a.ustart[m] = units; units += (O[m] + MR - 1) / MR;
    }
    a.ustart[n] = units;
    const size_t smem = (size_t)xoff;
    auto k = q8_multi_kernel;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q8_multi: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    if (cached_per_sm[dev] < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "q8_multi: kernel does not fit (smem %zu)", smem);
    int ctas = sms * cached_per_sm[dev];
    if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
    CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
    return 0;
}
