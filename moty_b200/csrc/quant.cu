// quant.cu -- activation quantizers (per row, per group of 32) and the load-time
// weight quantizers, bit-exact with the CPU code they replace.
#include "kernels.cuh"

// ---------------------------------------------------------------------------
// moty_hw_qrow_i8 (hw/hw_quant.h:9-16): one CTA per row.
// amax is order independent, so a parallel max is exact.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_max_256(float v, float *red) {
    v = warp_max_f32(v);
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float m = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) m = fmaxf(m, red[i]);
    __syncthreads();
    return m;
}

__global__ void __launch_bounds__(256) qrow_i8_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                                      float *__restrict__ scale, int n) {
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    const float *xr = x + row * n;
    int8_t *qr = q + row * n;
    const bool vec = (n % 4 == 0) && ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(qr) & 3) == 0);
    float amax = 0.f;
    if (vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
        for (int i = threadIdx.x; i < n / 4; i += 256) {
            float4 v = x4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 256) amax = fmaxf(amax, fabsf(xr[i]));
    }
    amax = block_max_256(amax, red);
    const float s = quant_scale(amax, 1e-12f);
    const float inv = __fdiv_rn(1.f, s);
    if (vec) {
        const float4 *x4 = reinterpret_cast<const float4 *>(xr);
        int *q4 = reinterpret_cast<int *>(qr);
        for (int i = threadIdx.x; i < n / 4; i += 256) {
            float4 v = x4[i];
            int a = quant_code(v.x, inv) & 255, b = quant_code(v.y, inv) & 255;
            int c = quant_code(v.z, inv) & 255, d = quant_code(v.w, inv) & 255;
            q4[i] = a | (b << 8) | (c << 16) | (d << 24);
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 256) qr[i] = (int8_t)quant_code(xr[i], inv);
    }
    if (threadIdx.x == 0) scale[row] = s;
}

// One routed token per CTA: quantize its row once (moty_hw_qrow_i8) and write the codes and the scale to every
// position the routing plan gave its K selections in the per-expert gathered batch (pos_of[s*K + k], -1 = the
// expert lives on another GPU).  This is the gather of nn/moe.c:172-186 folded into the row quantizer: the grouped
// tensor-core products then read contiguous rows per expert.
__global__ void __launch_bounds__(256) qrow_i8_scatter_kernel(const float *__restrict__ x, const int *__restrict__ pos_of, int K,
                                                              int8_t *__restrict__ xg, float *__restrict__ sxg, int n) {
    __shared__ float red[8];
    __shared__ int pos_s[64];
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    const float4 *x4 = reinterpret_cast<const float4 *>(x + row * n);
    if (threadIdx.x < K) pos_s[threadIdx.x] = pos_of[row * K + threadIdx.x];
    float amax = 0.f;
    for (int i = threadIdx.x; i < n / 4; i += 256) {
        float4 v = x4[i];
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    amax = block_max_256(amax, red);
    const float s = quant_scale(amax, 1e-12f);
    const float inv = __fdiv_rn(1.f, s);
    for (int i = threadIdx.x; i < n / 4; i += 256) {
        float4 v = x4[i];
        int a = quant_code(v.x, inv) & 255, b = quant_code(v.y, inv) & 255;
        int c = quant_code(v.z, inv) & 255, d = quant_code(v.w, inv) & 255;
        const int word = a | (b << 8) | (c << 16) | (d << 24);
        for (int k = 0; k < K; k++) {
            const int p = pos_s[k];
            if (p >= 0) reinterpret_cast<int *>(xg + (size_t)p * n)[i] = word;
        }
    }
    if (threadIdx.x < K && pos_s[threadIdx.x] >= 0) sxg[pos_s[threadIdx.x]] = s;
}

// n % 4 == 0, x rows 16-byte aligned, K <= 64
int launch_qrow_i8_scatter(const float *x, const int *pos_of, int S, int K, int8_t *xg, float *sxg, int n, cudaStream_t st) {
    if (S <= 0) return 0;
    CK(moty_launch_pdl(qrow_i8_scatter_kernel, dim3(S), dim3(256), (size_t)0, st, x, pos_of, K, xg, sxg, n));
    return 0;
}

// qrow_i8 over the first *nrows_dev rows only (a count the routing plan left on the device)
__global__ void __launch_bounds__(256) qrow_i8_counted_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                                              float *__restrict__ scale, int n, const int *__restrict__ nrows_dev) {
    __shared__ float red[8];
    pdl_trigger();
    pdl_wait();
    const size_t row = blockIdx.x;
    if ((int)row >= *nrows_dev) return;
    const float4 *x4 = reinterpret_cast<const float4 *>(x + row * n);
    float amax = 0.f;
    for (int i = threadIdx.x; i < n / 4; i += 256) {
        float4 v = x4[i];
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    amax = block_max_256(amax, red);
    const float s = quant_scale(amax, 1e-12f);
    const float inv = __fdiv_rn(1.f, s);
    int *q4 = reinterpret_cast<int *>(q + row * n);
    for (int i = threadIdx.x; i < n / 4; i += 256) {
        float4 v = x4[i];
        int a = quant_code(v.x, inv) & 255, b = quant_code(v.y, inv) & 255;
        int c = quant_code(v.z, inv) & 255, d = quant_code(v.w, inv) & 255;
        q4[i] = a | (b << 8) | (c << 16) | (d << 24);
    }
    if (threadIdx.x == 0) scale[row] = s;
}

int launch_qrow_i8_counted(const float *x, int8_t *q, float *scale, int rows_max, int n, const int *nrows_dev, cudaStream_t st) {
    if (rows_max <= 0) return 0;
    CK(moty_launch_pdl(qrow_i8_counted_kernel, dim3(rows_max), dim3(256), (size_t)0, st, x, q, scale, n, nrows_dev));
    return 0;
}

int launch_qrow_i8(const float *x, int8_t *q, float *scale, int rows, int n, cudaStream_t st) {
    if (rows <= 0 || n <= 0) return 0;
    CK(moty_launch_pdl(qrow_i8_kernel, dim3(rows), dim3(256), (size_t)0, st, x, q, scale, n));
    return 0;
}

// ---------------------------------------------------------------------------
// moty_hw_quant_g32 (hw/hw_q4r4.h:36-45): one warp per group, lane = element.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quant_g32_kernel(const float *__restrict__ x, int8_t *__restrict__ xq,
                                                        float *__restrict__ xs, int32_t *__restrict__ xsum,
                                                        long long ngroups) {
    pdl_trigger();
    pdl_wait();
    long long g = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (g >= ngroups) return;
    int lane = threadIdx.x & 31;
    float v = x[g * 32 + lane];
    float amax = warp_max_f32(fabsf(v));
    float s = quant_scale(amax, 1e-30f);
    float inv = __fdiv_rn(1.f, s);
    int c = quant_code(v, inv);
    xq[g * 32 + lane] = (int8_t)c;
    int total = warp_sum_i32(c);
    if (lane == 0) { xs[g] = s; xsum[g] = total; }
}

int launch_quant_g32(const float *x, int rows, int I, int8_t *xq, float *xs, int32_t *xsum, cudaStream_t st) {
    long long ng = (long long)rows * (I / 32);
    if (ng <= 0) return 0;
    CK(moty_launch_pdl(quant_g32_kernel, dim3((unsigned)((ng + 7) / 8)), dim3(256), (size_t)0, st, x, xq, xs, xsum, ng));
    return 0;
}

// ---------------------------------------------------------------------------
// moty_quantize_rows with bits = 8 (nn/quant.c:12-33): true division per element.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float *__restrict__ w, int8_t *__restrict__ q,
                                                            float *__restrict__ scale, int I) {
    __shared__ float red[8];
    const size_t row = blockIdx.x;
    const float *wr = w + row * I;
    int8_t *qr = q + row * I;
    float amax = 0.f;
    for (int i = threadIdx.x; i < I; i += 256) amax = fmaxf(amax, fabsf(wr[i]));
    amax = block_max_256(amax, red);
    float s = __fdiv_rn(amax, 127.f);
    if (s < 1e-8f) s = 1e-8f;
    for (int i = threadIdx.x; i < I; i += 256) {
        int v = __float2int_rn(__fdiv_rn(wr[i], s));
        v = v > 127 ? 127 : v;
        v = v < -128 ? -128 : v;
        qr[i] = (int8_t)v;
    }
    if (threadIdx.x == 0) scale[row] = s;
}

int launch_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I, cudaStream_t st) {
    if (O <= 0 || I <= 0) return 0;
    quantize_rows_kernel<<<O, 256, 0, st>>>(w, q, scale, I);
    CK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// moty_pack_q4r4_block (nn/quant.c:157-179): one warp per (row, group).
// The group's first largest-magnitude weight decides the sign of the step; the
// step is rounded to f16 and the codes are taken from the rounded step.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pack_q4r4_kernel(const float *__restrict__ w, int O, int I,
                                                        uint8_t *__restrict__ q4, uint16_t *__restrict__ s16) {
    const int nb = I / 32;
    const int O4 = (O + 3) / 4 * 4;
    long long task = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (task >= (long long)O4 * nb) return;
    int row = (int)(task / nb), g = (int)(task % nb), lane = threadIdx.x & 31;
    int blk = row >> 2, r = row & 3;
    uint8_t *dst = q4 + ((size_t)blk * nb + g) * 64 + r * 16;
    uint16_t *dd = s16 + ((size_t)blk * nb + g) * 4 + r;
    if (row >= O) {                       // padding row of the last block
        if (lane < 16) dst[lane] = 0x88;
        if (lane == 0) *dd = 0;
        return;
    }
    float v = w[(size_t)row * I + g * 32 + lane];
    float a = fabsf(v);
    // first lane holding the largest |v| (strict > in a sequential scan keeps the first)
    float m = warp_max_f32(a);
    unsigned who = __ballot_sync(0xffffffffu, a == m);
    int src = __ffs(who) - 1;
    float big = __shfl_sync(0xffffffffu, v, src);
    if (m == 0.f) big = 0.f;              // nothing exceeded |0|: the scan keeps its initial 0
    float other = ((v > 0.f) != (big > 0.f)) ? a : 0.f;
    other = warp_max_f32(other);
    float step = fmaxf(__fdiv_rn(fabsf(big), 8.f), __fdiv_rn(other, 7.f));
    __half h = __float2half_rn(big > 0.f ? -step : step);
    float dq = __half2float(h);
    float inv = dq != 0.f ? __fdiv_rn(1.f, dq) : 0.f;
    int c = __float2int_rn(__fmul_rn(v, inv));
    c = c < -8 ? -8 : c;
    c = c > 7 ? 7 : c;
    c += 8;
    int hi = __shfl_down_sync(0xffffffffu, c, 16);
    if (lane < 16) dst[lane] = (uint8_t)(c | (hi << 4));
    if (lane == 0) *dd = __half_as_ushort(h);
}

int launch_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16, cudaStream_t st) {
    if (O <= 0 || I < 32) return 0;
    long long tasks = (long long)((O + 3) / 4 * 4) * (I / 32);
    pack_q4r4_kernel<<<(unsigned)((tasks + 7) / 8), 256, 0, st>>>(w, O, I, q4, s16);
    CK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// Per-row int4 rows (element 2j in the low nibble, 2j + 1 in the high one; hw/hw_scalar.h:14-22) -> signed int8 codes
// nibble - 8, rows of n codes from rows of (n + 1) / 2 bytes.  The integer dot over these codes IS the reference's
// dot_i4i8 / dot_i4i8p sum (hw/hw_avx512.h:106-145), so an int4 expert stored this way runs through the int8 kernels
// with the reference's bits.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) i4_rows_to_i8_kernel(const uint8_t *__restrict__ q4, int8_t *__restrict__ q8, long long rows, int n) {
    const int rb = (n + 1) / 2;
    const long long total = rows * (long long)n;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
        const long long r = i / n; const int j = (int)(i - r * n);
        const uint8_t b = q4[r * rb + (j >> 1)];
        q8[i] = (int8_t)(((j & 1) ? (b >> 4) : (b & 15)) - 8);
    }
}

int launch_i4_rows_to_i8(const uint8_t *q4, int8_t *q8, long long rows, int n, cudaStream_t st) {
    if (rows <= 0 || n <= 0) return 0;
    long long blocks = (rows * (long long)n + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    i4_rows_to_i8_kernel<<<(unsigned)blocks, 256, 0, st>>>(q4, q8, rows, n);
    CK(cudaGetLastError());
    return 0;
}
