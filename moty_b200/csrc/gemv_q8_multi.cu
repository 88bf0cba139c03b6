// gemv_q8_multi.cu -- several independent Q8_0 decode products in ONE launch.
//
// A decode step is full of small matrices whose own GEMV launch costs more than their bytes: a 1-3 MB matrix is
// 0.2-0.5 us of HBM time behind 4-5 us of launch, prologue and tail.  This kernel takes up to eight (matrix, row)
// pairs -- moty_matmul_q_s with S = 1 for each (nn/matmul.c:51-66, IDOT=1), e.g. the q, k and v projections of a
// layer, or independent products of a benchmark pass -- cuts ALL their rows into units of two, four or eight rows (16
// 128-bit loads per lane in flight whatever the row length) and deals the units round-robin to one persistent grid, so
// the fixed cost is paid once and the tail is one unit long.
// Every CTA quantizes each activation row (moty_hw_qrow_i8, hw/hw_quant.h:9-16: exact amax, true division,
// round-half-even) into shared memory behind its first weight loads.
// Same dp4a arithmetic and the same (scale[o] * sx) * (float)dot epilogue as q8_stream_kernel: same bits.
// Rows longer than 4096 values are split in K like the single-matrix kernel's: a unit is two rows x one segment of at
// most 4 KB, the exact int32 partial dots of a row meet in a 64-bit cell (arrival count || biased sum) by one atomic
// each, and the lane that brings the last part writes the f32 result and re-zeroes the cell.
// Limits: I a multiple of 16, I <= 16384, x 16-byte aligned; cells (zero between launches) for matrices with I > 4096.
#include "kernels.cuh"
#include <string.h>

namespace {

constexpr int MULTI_MAX = 8;

// N per-lane partial sums -> lane L holds the total of value (L >> (5 - log2 N))
template <int N> struct LgM { static constexpr int v = 1 + LgM<N / 2>::v; };
template <> struct LgM<1> { static constexpr int v = 0; };
template <int N>
__device__ __forceinline__ void reduce_multi_m(int (&v)[N], int lane) {
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) {
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            const bool up = (lane & off) != 0;
            const int send = up ? v[i] : v[i + n / 2];
            const int keep = up ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

// A unit is R rows of one matrix with LPR 128-bit loads per lane and row, R * LPR = 16 loads in flight per lane whatever
// the row length: rows of up to 1024 values go eight to a unit (kind 2), up to 2048 four (kind 1), longer ones two (kind 0).
struct MultiArgs {
    const int8_t *w[MULTI_MAX]; const float *scale[MULTI_MAX]; const float *x[MULTI_MAX]; float *y[MULTI_MAX];
    int O[MULTI_MAX], I16[MULTI_MAX], xoff[MULTI_MAX];     // xoff: where matrix m's codes start in shared memory (bytes)
    int kind[MULTI_MAX];                                   // 3: rows longer than 4096 values, split in K
    int KS[MULTI_MAX], seg[MULTI_MAX];                     // kind 3: segments per row, int4s per segment
    unsigned long long *cell[MULTI_MAX];                   // kind 3: one cell per output row, all zero between launches
    int ustart[MULTI_MAX + 1];                             // prefix of units per matrix
    int n;
};

template <int R, int LPR>
__device__ __forceinline__ void multi_issue(const MultiArgs &a, int m, int r0, int lane, int4 (&wv)[16], float &my_scale,
                                            int k0 = 0, int kend = 1 << 30) {
    const int I16 = a.I16[m], O = a.O[m];
    kend = kend < I16 ? kend : I16;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int o = r0 + r < O ? r0 + r : O - 1;
        const int4 *p = reinterpret_cast<const int4 *>(a.w[m]) + (size_t)o * I16;
#pragma unroll
        for (int j = 0; j < LPR; j++) {
            const int k = k0 + j * 32 + lane;
            wv[r * LPR + j] = k < kend ? ldg_stream16(p + k) : make_int4(0, 0, 0, 0);
        }
    }
    constexpr int SH = 5 - LgM<R>::v;                       // after the reduction lane L reports row L >> SH
    const int o = r0 + (lane >> SH);
    my_scale = __ldg(a.scale[m] + (o < O ? o : O - 1));
}

template <int R, int LPR>
__device__ __forceinline__ void multi_dots(const MultiArgs &a, int m, int lane, const int4 (&wv)[16], const int4 *xs, int (&dot)[8],
                                           int k0 = 0) {
    const int I16 = a.I16[m];
#pragma unroll
    for (int r = 0; r < 8; r++) dot[r] = 0;
#pragma unroll
    for (int j = 0; j < LPR; j++) {
        if (k0 + j * 32 < I16) {                           // warp-uniform
            int k = k0 + j * 32 + lane; k = k < I16 ? k : I16 - 1;     // weights past the row or the segment were loaded as zeros
            const int4 xv = xs[k];
#pragma unroll
            for (int r = 0; r < R; r++) dot[r] = dp4a4(wv[r * LPR + j], xv, dot[r]);
        }
    }
}

template <int R>
__device__ __forceinline__ void multi_write(const MultiArgs &a, int m, int r0, int lane, int (&dot)[8], float my_scale, float sx) {
    int d[R];
#pragma unroll
    for (int r = 0; r < R; r++) d[r] = dot[r];
    reduce_multi_m<R>(d, lane);
    constexpr int SH = 5 - LgM<R>::v;
    const int o = r0 + (lane >> SH);
    // (scale[o] * sx) * (float)dot, left to right (nn/matmul.c:34)
    if ((lane & ((1 << SH) - 1)) == 0 && o < a.O[m]) a.y[m][o] = __fmul_rn(__fmul_rn(my_scale, sx), (float)d[0]);
}

// kind 3: the two rows' partial dots of one segment go to their cells; the last arrival owns the cell
__device__ __forceinline__ void multi_write_split(const MultiArgs &a, int m, int r0, int lane, int (&dot)[8], float my_scale, float sx) {
    int d[2] = {dot[0], dot[1]};
    reduce_multi_m<2>(d, lane);
    const int o = r0 + (lane >> 4), KS = a.KS[m];
    if ((lane & 15) == 0 && o < a.O[m]) {
        const unsigned long long bias = 1ull << 33;
        const unsigned long long add = (1ull << 40) + (unsigned long long)((long long)d[0] + (long long)bias);
        unsigned long long *cell = a.cell[m] + o;
        const unsigned long long old = atomicAdd(cell, add);
        if ((int)(old >> 40) == KS - 1) {
            const long long sum = (long long)((old + add) & ((1ull << 40) - 1)) - (long long)KS * (long long)bias;
            *cell = 0ull;
            a.y[m][o] = __fmul_rn(__fmul_rn(my_scale, sx), (float)(int)sum);
        }
    }
}

__device__ __forceinline__ int multi_rows(int kind) { return kind == 2 ? 8 : (kind == 1 ? 4 : 2); }

__global__ void __launch_bounds__(256, 2) q8_multi_kernel(MultiArgs a) {
    extern __shared__ int4 smem4[];
    __shared__ float red[8];
    __shared__ float sx_s[MULTI_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nunits = a.ustart[a.n], nwarps = gridDim.x * 8;
    int8_t *xq_s = reinterpret_cast<int8_t *>(smem4);

    int4 wv[16];
    float my_scale = 0.f;
    int um = 0, ur = 0, uk = 0;                            // matrix, first row and first int4 of the unit in flight
    auto issue = [&](int u) {
        int m = 0;
        while (m + 1 < a.n && u >= a.ustart[m + 1]) m++;
        const int kind = a.kind[m];
        um = m; uk = 0;
        if (kind == 3) {                                   // unit = (row pair, segment); a row's segments go to neighbouring warps
            const int uu = u - a.ustart[m], rg = uu / a.KS[m], ks = uu - rg * a.KS[m];
            ur = rg * 2; uk = ks * a.seg[m];
            multi_issue<2, 8>(a, m, ur, lane, wv, my_scale, uk, uk + a.seg[m]);
            return;
        }
        ur = (u - a.ustart[m]) * multi_rows(kind);
        if (kind == 2) multi_issue<8, 2>(a, m, ur, lane, wv, my_scale);
        else if (kind == 1) multi_issue<4, 4>(a, m, ur, lane, wv, my_scale);
        else multi_issue<2, 8>(a, m, ur, lane, wv, my_scale);
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
        const int m = um, r0 = ur, k0 = uk, kind = a.kind[m];
        const int4 *xs = reinterpret_cast<const int4 *>(xq_s + a.xoff[m]);
        const float sx = sx_s[m], sc = my_scale;
        int dot[8];
        if (kind == 3) multi_dots<2, 8>(a, m, lane, wv, xs, dot, k0);
        else if (kind == 2) multi_dots<8, 2>(a, m, lane, wv, xs, dot);
        else if (kind == 1) multi_dots<4, 4>(a, m, lane, wv, xs, dot);
        else multi_dots<2, 8>(a, m, lane, wv, xs, dot);
        u += nwarps;
        if (u < nunits) issue(u);                          // the next unit's loads go out before this result is written
        if (kind == 3) multi_write_split(a, m, r0, lane, dot, sc, sx);
        else if (kind == 2) multi_write<8>(a, m, r0, lane, dot, sc, sx);
        else if (kind == 1) multi_write<4>(a, m, r0, lane, dot, sc, sx);
        else multi_write<2>(a, m, r0, lane, dot, sc, sx);
    }
}

}  // namespace

bool q8_multi_supported(int I) { return I % 16 == 0 && I >= 16 && I <= MOTY_QROW_MAX; }

// cells: for every matrix with I > 4096, O[m] zeroed 64-bit words (null otherwise); they are zero again when the launch ends
int launch_q8_multi(int n, const int8_t *const *w, const float *const *scale, const float *const *x, float *const *y,
                    const int *O, const int *I, int sms, cudaStream_t st, unsigned long long *const *cells) {
    if (n < 1 || n > MULTI_MAX) return moty_set_error(MOTY_CUDA_EARG, "q8_multi: %d matrices (1..%d)", n, MULTI_MAX);
    MultiArgs a;
    memset(&a, 0, sizeof a);
    a.n = n;
    int units = 0, xoff = 0;
    for (int m = 0; m < n; m++) {
        if (!q8_multi_supported(I[m]) || O[m] < 1 || (reinterpret_cast<uintptr_t>(x[m]) & 15))
            return moty_set_error(MOTY_CUDA_EARG, "q8_multi: matrix %d is %dx%d (rows of 16..%d bytes, x 16-byte aligned)", m, O[m], I[m], MOTY_QROW_MAX);
        a.w[m] = w[m]; a.scale[m] = scale[m]; a.x[m] = x[m]; a.y[m] = y[m]; a.O[m] = O[m]; a.I16[m] = I[m] / 16;
        a.xoff[m] = xoff; xoff += I[m];
        a.kind[m] = I[m] <= 1024 ? 2 : (I[m] <= 2048 ? 1 : (I[m] <= 4096 ? 0 : 3));
        if (a.kind[m] == 3) {
            if (!cells || !cells[m]) return moty_set_error(MOTY_CUDA_EARG, "q8_multi: K-split cells missing for matrix %d", m);
            const int I16 = I[m] / 16;
            a.KS[m] = (I16 + 255) / 256;                   // segments of at most 4 KB
            a.seg[m] = (I16 + a.KS[m] - 1) / a.KS[m];
            a.cell[m] = cells[m];
            a.ustart[m] = units; units += ((O[m] + 1) / 2) * a.KS[m];
            continue;
        }
        const int rows = a.kind[m] == 2 ? 8 : (a.kind[m] == 1 ? 4 : 2);
        a.ustart[m] = units; units += (O[m] + rows - 1) / rows;
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
