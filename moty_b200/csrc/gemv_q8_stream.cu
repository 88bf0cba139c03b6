// gemv_q8_stream.cu -- the decode GEMV: Q8_0 weights streamed at HBM speed for
// 1..8 activation rows.  Replaces moty_matmul_q_s (nn/matmul.c:51-66, IDOT=1).
//
// Persistent grid (as many CTAs as fit per SM).  The matrix is cut into UNITS of
// about 4 KB: R rows x one K segment, dealt round-robin to the warps, so every
// warp streams for the whole launch and the tail is one unit long whatever the
// shape.  A unit is fetched with R*LPR independent 128-bit L1-bypassing loads
// per lane, all issued before anything is consumed, and the next unit's loads
// go out before the current result is written.
// The activation row is quantized by each CTA (moty_hw_qrow_i8,
// hw/hw_quant.h:9-16) while its warps' first loads are already in flight.
//
// Rows longer than 4 KB are split in K: the int32 partial dots of a row are
// added into a global cell (exact, order independent) and the lane that brings
// the last part writes the f32 result and re-zeroes the cell.
#include "kernels.cuh"
#include "resnorm.cuh"

struct StreamArgs {
    const int8_t *w; const float *scale;
    const float *x;                 // FUSED: f32 row
    const float *t, *g; float *xout; float eps;   // FUSED, optional: the row is rmsnorm(x + t) * g, and x + t goes to xout
    const float *gt;                              // FUSED == 2: the sandwich form, x + rmsnorm(t) * gt in place of x + t
    const int8_t *xi; const float *sx;   // not fused: quantized rows [S][I] and their scales
    float *y; int32_t *acc_out;     // [S][O]
    unsigned long long *cell;       // K-split cells [S][O], all 0 between launches
    int S, I, O, KS, seg;           // seg = int4s per K segment
};

template <int N> struct Lg { static constexpr int v = 1 + Lg<N / 2>::v; };
template <> struct Lg<1> { static constexpr int v = 0; };

template <int N>
__device__ __forceinline__ void reduce_multi(int (&v)[N], int lane) {
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) {
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            bool up = (lane & off) != 0;
            int send = up ? v[i] : v[i + n / 2];
            int keep = up ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

// FUSED: 0 = quantized rows come in; 1 = one f32 row, quantized here (optionally after x + t and the RMS norm);
// 2 = the same with gemma's sandwich step in front (resnorm.cuh) -- its own instantiation, so that the common ones keep
// their register budget
template <int NS, int R, int LPR, int FUSED>
__global__ void __launch_bounds__(256, (NS <= 2 ? 4 : 2)) q8_stream_kernel(StreamArgs a) {
    extern __shared__ int4 smem4[];
    __shared__ float red[8];
    __shared__ float sx_s[NS];
    __shared__ double red64[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int I = a.I, I16 = I / 16, O = a.O, KS = a.KS, SEG = a.seg;
    const int nrg = (O + R - 1) / R;
    const int nunits = nrg * KS;
    constexpr int SH = 5 - Lg<R * NS>::v;          // lanes sharing one reduced value
    const int my = lane >> SH;                     // the (row, token) this lane reports: r = my / NS, s = my % NS
    const int my_r = my / NS;

    int4 wv[R][LPR];
    float my_scale = 0.f;
    auto issue = [&](int t) {
        int rg = t / KS, ks = t - rg * KS;
        int k0 = ks * SEG, kend = k0 + SEG < I16 ? k0 + SEG : I16;
#pragma unroll
        for (int r = 0; r < R; r++) {
            int o = rg * R + r < O ? rg * R + r : O - 1;
            const int4 *p = reinterpret_cast<const int4 *>(a.w) + (size_t)o * I16;
#pragma unroll
            for (int j = 0; j < LPR; j++) {
                int k = k0 + j * 32 + lane;
                wv[r][j] = k < kend ? ldg_stream16(p + k) : make_int4(0, 0, 0, 0);
            }
        }
        int o = rg * R + my_r;
        my_scale = __ldg(a.scale + (o < O ? o : O - 1));
    };
    // static round-robin over the persistent warps: every warp streams the whole time and the
    // launch ends within one unit of the others (a shared ticket counter was measured slower:
    // tens of thousands of atomics on one address serialise in L2)
    const int nwarps = gridDim.x * 8;
    int t0 = blockIdx.x * 8 + warp;
    pdl_trigger();
    if (t0 < nunits) issue(t0);          // weights only: may run before the previous kernel has finished
    pdl_wait();                          // activations and outputs from here on

    // ---- activation rows into shared memory (int8 codes) ----
    int8_t *xq_s = reinterpret_cast<int8_t *>(smem4);
    if (FUSED) {
        // short rows keep an f32 copy in shared memory between the two passes; long rows are
        // re-read from L2 instead so that four CTAs still fit on an SM
        const bool stage = I <= 4096;
        float *xf = reinterpret_cast<float *>(xq_s + I);
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
        float amax = 0.f;
        if (FUSED == 2) {
            amax = resnorm_row(a.x, a.t, a.gt, a.g, a.xout, a.eps, I, xf, red64, red, blockIdx.x == 0);
        } else if (a.t) {
            // residual add and RMS norm first (hw/hw_ops.h:30-32 and 14-18), element for element and sum for sum as the
            // separate add+norm launch does them, so both routes give the same bits.  Every CTA forms the row for
            // itself; CTA 0 also writes the sum out (to another buffer: the others are still reading x).  I <= 4096.
            // Loads go out four rounds at a time (a row of 1024 is one round trip), the gains of the first four with them.
            double ms = 0;
            float gv[4];
#pragma unroll
            for (int j = 0; j < 4; j++) { const int i = threadIdx.x + 256 * j; gv[j] = i < I ? a.g[i] : 0.f; }
            for (int i0 = threadIdx.x; i0 < I; i0 += 1024) {
                float xv[4], tv[4];
#pragma unroll
                for (int j = 0; j < 4; j++) { const int i = i0 + 256 * j; xv[j] = i < I ? a.x[i] : 0.f; tv[j] = i < I ? a.t[i] : 0.f; }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int i = i0 + 256 * j;
                    if (i < I) {
                        const float v = __fadd_rn(xv[j], tv[j]);
                        xf[i] = v;
                        if (blockIdx.x == 0) a.xout[i] = v;
                        ms += (double)v * (double)v;
                    }
                }
            }
            for (int off = 16; off > 0; off >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, off);
            if (lane == 0) red64[warp] = ms;
            __syncthreads();
            ms = 0;
            for (int i = 0; i < 8; i++) ms += red64[i];
            const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / I), a.eps)));
            for (int i0 = threadIdx.x; i0 < I; i0 += 1024) {
                if (i0 >= 1024) {
#pragma unroll
                    for (int j = 0; j < 4; j++) { const int i = i0 + 256 * j; gv[j] = i < I ? a.g[i] : 0.f; }
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
        } else
        for (int i = threadIdx.x; i < I / 4; i += 256) {
            float4 v = x4[i];
            if (stage) reinterpret_cast<float4 *>(xf)[i] = v;
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        amax = warp_max_f32(amax);
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
        const float sx = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, sx);
        int *xq = reinterpret_cast<int *>(xq_s);
        for (int i = threadIdx.x; i < I / 4; i += 256) {
            float4 v = stage ? reinterpret_cast<const float4 *>(xf)[i] : x4[i];
            int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
            int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
            xq[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        if (threadIdx.x == 0) sx_s[0] = sx;
    } else {
        for (int idx = threadIdx.x; idx < NS * I16; idx += 256) {
            int s = idx / I16, k = idx - s * I16;
            smem4[idx] = s < a.S ? reinterpret_cast<const int4 *>(a.xi + (size_t)s * I)[k] : make_int4(0, 0, 0, 0);
        }
        if (threadIdx.x < NS) sx_s[threadIdx.x] = threadIdx.x < a.S ? a.sx[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const int my_s = my % NS;
    const float my_sx = sx_s[my_s];

    while (t0 < nunits) {
        const int rg = t0 / KS, ks = t0 - rg * KS;
        const int k0 = ks * SEG;
        int flat[R * NS];
#pragma unroll
        for (int i = 0; i < R * NS; i++) flat[i] = 0;
#pragma unroll
        for (int j = 0; j < LPR; j++) {
            int k = k0 + j * 32 + lane;
            k = k < I16 ? k : I16 - 1;             // weights beyond the segment were loaded as zeros
#pragma unroll
            for (int s = 0; s < NS; s++) {
                int4 xv = smem4[s * I16 + k];
#pragma unroll
                for (int r = 0; r < R; r++) flat[r * NS + s] = dp4a4(wv[r][j], xv, flat[r * NS + s]);
            }
        }
        reduce_multi<R * NS>(flat, lane);
        const float sc = my_scale;
        const int o = rg * R + my_r;
        // next unit's loads go out before this unit's result is written
        t0 += nwarps;
        if (t0 < nunits) issue(t0);
        const bool reporter = (lane & ((1 << SH) - 1)) == 0 && o < O && my_s < a.S;
        if (KS == 1) {
            if (reporter) {
                // (scale[o] * sx[s]) * (float)dot, left to right (nn/matmul.c:34)
                a.y[(size_t)my_s * O + o] = __fmul_rn(__fmul_rn(sc, my_sx), (float)flat[0]);
                if (a.acc_out) a.acc_out[(size_t)my_s * O + o] = flat[0];
            }
        } else {
            // K-split: one 64-bit cell per (token, row) holds the arrival count (bits 40..) and
            // the biased sum of the exact int32 parts (bits 0..39).  One atomic both adds and
            // tells the last arrival, which then owns the cell: it writes y and re-zeroes it.
            if (reporter) {
                const unsigned long long bias = 1ull << 33;
                unsigned long long add = (1ull << 40) + (unsigned long long)((long long)flat[0] + (long long)bias);
                unsigned long long *cell = a.cell + (size_t)my_s * O + o;
                unsigned long long old = atomicAdd(cell, add);
                if ((int)(old >> 40) == KS - 1) {
                    long long sum = (long long)((old + add) & ((1ull << 40) - 1)) - (long long)KS * (long long)bias;
                    int total = (int)sum;
                    *cell = 0ull;
                    a.y[(size_t)my_s * O + o] = __fmul_rn(__fmul_rn(sc, my_sx), (float)total);
                    if (a.acc_out) a.acc_out[(size_t)my_s * O + o] = total;
                }
            }
        }
    }
}

template <int NS, int R, int LPR, int FUSED>
static int launch_t(const StreamArgs &a, int sms, cudaStream_t st) {
    size_t smem = FUSED ? (a.I <= 4096 ? (size_t)a.I * 5 : (size_t)a.I) : (size_t)NS * a.I;
    auto k = q8_stream_kernel<NS, R, LPR, FUSED>;
    // the occupancy query costs a few microseconds of host time: remember the last answer
    // (all GPUs a process drives are the same model)
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q8_stream: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {                         // stored +1 so that zero-init means "nothing cached"
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    int per_sm = cached_per_sm[dev];
    if (per_sm < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "q8_stream: kernel does not fit (smem %zu)", smem);
    int nunits = ((a.O + R - 1) / R) * a.KS;
    int ctas = sms * per_sm;
    if (ctas > (nunits + 7) / 8) ctas = (nunits + 7) / 8;        // never more warps than units
    CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
    return 0;
}

template <int NS, int FUSED>
static int launch_ns(const StreamArgs &a, int lpr, int sms, cudaStream_t st) {
    if (lpr <= 2) return launch_t<NS, 4, 2, FUSED>(a, sms, st);
    if (lpr <= 4) return launch_t<NS, 2, 4, FUSED>(a, sms, st);
    return launch_t<NS, 1, 8, FUSED>(a, sms, st);
}

// x: f32 rows (S == 1 is quantized inside the kernel); xi/sx: the quantized rows for S > 1.
// counters: 2 ints (ticket, done), zero between launches; cell: K-split cells [S][O] (zero
// between launches) or null when I <= 4096.
int launch_q8_stream(const int8_t *w, const float *scale, const float *x, const int8_t *xi, const float *sx,
                     float *y, int32_t *acc, int S, int I, int O, int *counters, unsigned long long *cell,
                     int sms, cudaStream_t st, const float *t, const float *g, float *xout, float eps, const float *gt) {
    if (I % 16 != 0 || I > MOTY_QROW_MAX || S < 1 || S > 8) return moty_set_error(MOTY_CUDA_EARG, "q8_stream: S=%d I=%d", S, I);
    if (t && (S != 1 || !x || !g || !xout || xout == x || I > 4096))
        return moty_set_error(MOTY_CUDA_EARG, "q8_stream: add+norm wants one f32 row of at most 4096 values and its own output");
    if (O <= 0) return 0;
    StreamArgs a;
    a.w = w; a.scale = scale; a.x = x; a.xi = xi; a.sx = sx; a.y = y; a.acc_out = acc;
    a.t = t; a.g = g; a.xout = xout; a.eps = eps; a.gt = t ? gt : nullptr;
    a.cell = cell; (void)counters;
    a.S = S; a.I = I; a.O = O;
    int I16 = I / 16;
    a.KS = (I16 + 255) / 256;                        // segments of at most 4 KB
    a.seg = (I16 + a.KS - 1) / a.KS;
    if (a.KS > 1 && !cell) return moty_set_error(MOTY_CUDA_EARG, "q8_stream: K-split cells missing");
    int lpr = (a.seg + 31) / 32;                     // 128-bit loads per lane and row
    if (S == 1 && x && a.gt) return launch_ns<1, 2>(a, lpr, sms, st);   // f32 row behind gemma's sandwich step
    if (S == 1 && x) return launch_ns<1, 1>(a, lpr, sms, st);        // f32 row: quantized inside the kernel
    if (S == 1) return launch_ns<1, 0>(a, lpr, sms, st);             // already quantized (tail of a chunked batch)
    if (S == 2) return launch_ns<2, 0>(a, lpr, sms, st);
    if (S <= 4) return launch_ns<4, 0>(a, lpr, sms, st);
    return launch_ns<8, 0>(a, lpr, sms, st);
}
