// norm.cu -- the small f32 steps of a decoder layer around the matmuls, so that a layer's
// activations can stay on the device: RMS norm of a row (moty_rmsnorm_row, nn/norm.c:7 ->
// moty_hw_rmsnorm_ref, hw/hw_ops.h:14-18), the residual add (moty_hw_add_ref, hw/hw_ops.h:30-32)
// and the int8 embedding row (embed_row, runtime/rt_model_load.h:656-660).
#include "kernels.cuh"

namespace {

// One CTA per row: x (+ t), mean of squares in double, r = 1 / sqrtf((float)(ms / n) + eps), out = (x * r) * w.
// Rows of up to 2048 values stay in registers and the gains are requested with them, so the kernel is one memory
// round trip; longer rows are re-read.  ADD: x += t first (hw/hw_ops.h:30-32), the sum is written back.
constexpr int NR_PER = 8;

template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(float *x, const float *t, float *out, const float *w, int D, float eps) {
    __shared__ double red[8];
    pdl_trigger();
    pdl_wait();
    float *xr = x + (size_t)blockIdx.x * D;
    const float *tr = ADD ? t + (size_t)blockIdx.x * D : nullptr;
    float *orow = out + (size_t)blockIdx.x * D;
    const bool in_regs = D <= 256 * NR_PER;
    float v[NR_PER], wv[NR_PER];
    double ms = 0;
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NR_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            v[j] = i < D ? xr[i] : 0.f;
            wv[j] = i < D ? w[i] : 0.f;
            if (ADD && i < D) v[j] = __fadd_rn(v[j], tr[i]);
        }
#pragma unroll
        for (int j = 0; j < NR_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            if (ADD && i < D) xr[i] = v[j];
            ms += (double)v[j] * (double)v[j];
        }
    } else {
        for (int i = threadIdx.x; i < D; i += 256) {
            float a = xr[i];
            if (ADD) { a = __fadd_rn(a, tr[i]); xr[i] = a; }
            ms += (double)a * (double)a;
        }
    }
    for (int off = 16; off > 0; off >>= 1) ms += __shfl_xor_sync(0xffffffffu, ms, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ms;
    __syncthreads();
    ms = 0;
    for (int i = 0; i < 8; i++) ms += red[i];
    const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / D), eps)));
    if (in_regs) {
#pragma unroll
        for (int j = 0; j < NR_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            if (i < D) orow[i] = __fmul_rn(__fmul_rn(v[j], r), wv[j]);
        }
    } else {
        for (int i = threadIdx.x; i < D; i += 256) orow[i] = __fmul_rn(__fmul_rn(xr[i], r), w[i]);   // the thread's own writes above
    }
}

// The sandwich step of engines/gemma.c:468-474 and :478-482, one CTA per row: tn = (t * r_t) * g1 (the norm of the
// block's output, in place there), x += tn, then -- when out is given -- out = (x * r_x) * g2, the norm that opens the
// next block.  Both means of squares in double as in gnorm_row (engines/gemma.c:279-284); the gains are the multipliers
// themselves (1 + w for a zero-centred checkpoint).  Rows of up to 4096 values stay in registers.
constexpr int NA_PER = 16;

__device__ __forceinline__ double block_sum_256(double v, double *red) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();                                          // red may still be read from a previous sum
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double s = 0;
    for (int i = 0; i < 8; i++) s += red[i];
    return s;
}

__global__ void __launch_bounds__(256) normadd_rmsnorm_rows_kernel(float *x, const float *t, const float *g1, float *out, const float *g2,
                                                                   int D, float eps) {
    __shared__ double red[8];
    pdl_trigger();
    pdl_wait();
    float *xr = x + (size_t)blockIdx.x * D;
    const float *tr = t + (size_t)blockIdx.x * D;
    float *orow = out ? out + (size_t)blockIdx.x * D : nullptr;
    if (D <= 256 * NA_PER) {
        float tv[NA_PER], xv[NA_PER], g1v[NA_PER], g2v[NA_PER];       // every load of the kernel goes out at once
        double ms = 0;
#pragma unroll
        for (int j = 0; j < NA_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            tv[j] = i < D ? tr[i] : 0.f;
            xv[j] = i < D ? xr[i] : 0.f;
            g1v[j] = i < D ? g1[i] : 0.f;
            g2v[j] = i < D && orow ? g2[i] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < NA_PER; j++) ms += (double)tv[j] * (double)tv[j];
        ms = block_sum_256(ms, red);
        const float rt = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / D), eps)));
        ms = 0;
#pragma unroll
        for (int j = 0; j < NA_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            if (i < D) {
                xv[j] = __fadd_rn(xv[j], __fmul_rn(__fmul_rn(tv[j], rt), g1v[j]));
                xr[i] = xv[j];
            }
            ms += (double)xv[j] * (double)xv[j];
        }
        if (!orow) return;
        ms = block_sum_256(ms, red);
        const float rx = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / D), eps)));
#pragma unroll
        for (int j = 0; j < NA_PER; j++) {
            const int i = threadIdx.x + 256 * j;
            if (i < D) orow[i] = __fmul_rn(__fmul_rn(xv[j], rx), g2v[j]);
        }
        return;
    }
    double ms = 0;
    for (int i = threadIdx.x; i < D; i += 256) ms += (double)tr[i] * (double)tr[i];
    ms = block_sum_256(ms, red);
    const float rt = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / D), eps)));
    ms = 0;
    for (int i = threadIdx.x; i < D; i += 256) {
        const float a = __fadd_rn(xr[i], __fmul_rn(__fmul_rn(tr[i], rt), g1[i]));
        xr[i] = a;
        ms += (double)a * (double)a;
    }
    if (!orow) return;
    ms = block_sum_256(ms, red);
    const float rx = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / D), eps)));
    for (int i = threadIdx.x; i < D; i += 256) orow[i] = __fmul_rn(__fmul_rn(xr[i], rx), g2[i]);   // the thread's own writes above
}

__global__ void __launch_bounds__(256) add_kernel(float *y, const float *x, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(y[i], x[i]);
}

// dst[s][i] = (qs[id] * scale) * (float)q[id][i]
__global__ void __launch_bounds__(256) embed_rows_kernel(float *dst, const int8_t *q, const float *qs, const int *ids, int D, int V,
                                                         float scale) {
    pdl_trigger();
    pdl_wait();
    int id = ids[blockIdx.x];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const float es = __fmul_rn(qs[id], scale);
    for (int i = threadIdx.x; i < D; i += 256) dst[(size_t)blockIdx.x * D + i] = __fmul_rn(es, (float)q[(size_t)id * D + i]);
}

}  // namespace

int launch_rmsnorm_rows(float *out, const float *x, const float *w, int S, int D, float eps, cudaStream_t st) {
    if (S <= 0) return 0;
    if (D <= 0) return moty_set_error(MOTY_CUDA_EARG, "rmsnorm: D=%d", D);
    CK(moty_launch_pdl(rmsnorm_rows_kernel<false>, dim3(S), dim3(256), (size_t)0, st, const_cast<float *>(x), (const float *)nullptr, out, w, D, eps));
    return 0;
}

int launch_add_rmsnorm_rows(float *x, const float *t, float *out, const float *w, int S, int D, float eps, cudaStream_t st) {
    if (S <= 0) return 0;
    if (D <= 0) return moty_set_error(MOTY_CUDA_EARG, "add_rmsnorm: D=%d", D);
    CK(moty_launch_pdl(rmsnorm_rows_kernel<true>, dim3(S), dim3(256), (size_t)0, st, x, t, out, w, D, eps));
    return 0;
}

int launch_normadd_rmsnorm_rows(float *x, const float *t, const float *g1, float *out, const float *g2, int S, int D, float eps,
                                cudaStream_t st) {
    if (S <= 0) return 0;
    if (D <= 0) return moty_set_error(MOTY_CUDA_EARG, "normadd_rmsnorm: D=%d", D);
    CK(moty_launch_pdl(normadd_rmsnorm_rows_kernel, dim3(S), dim3(256), (size_t)0, st, x, t, g1, out, g2, D, eps));
    return 0;
}

int launch_add(float *y, const float *x, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    CK(moty_launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, st, y, x, n));
    return 0;
}

int launch_embed_rows(float *dst, const int8_t *q, const float *qs, const int *ids, int S, int D, int V, float scale, cudaStream_t st) {
    if (S <= 0) return 0;
    CK(moty_launch_pdl(embed_rows_kernel, dim3(S), dim3(256), (size_t)0, st, dst, q, qs, ids, D, V, scale));
    return 0;
}
