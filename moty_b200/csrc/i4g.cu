// i4g.cu -- WF_I4G weights (grouped int4, group 32, f32 group scales, row-major nibbles): the reference's DEFAULT
// product for this layout.  (Its integer path, IDOT4=1, is in i4g_mma.cu for batches and q4r4_gemv2.cu for one row.)
#include "kernels.cuh"

// ---------------------------------------------------------------------------
// The reference's DEFAULT product for this layout (IDOT4 unset): f32 activations x dequantized int4, no activation
// quantizer (moty_matmul_i4_grouped_s -> i4g_f32_rows, nn/matmul.c:196-253).  Per group of 32:
//     a += (sum_j x[j] * (float)(nibble_j - 8)) * scale[o][g]
// in ascending group order.  A warp takes one weight row and up to four tokens; lane j owns element j of every group
// (its nibble and its x values), the 32 products of a group meet in a shuffle tree, lane 0 keeps the running sums.
// The sum inside a group is taken in the tree's order, the reference's in its SIMD tier's (_mm512_reduce_add_ps, or
// eight-lane FMA chains): agreement to f32 rounding of a 32-term sum, not bit for bit -- the reference's own tiers
// differ from each other in the same way.  A correct path for engines that run without IDOT4, not a tuned one.
// ---------------------------------------------------------------------------
template <int NS>
__global__ void __launch_bounds__(256) i4g_f32_rows_kernel(const uint8_t *__restrict__ w4, const float *__restrict__ scale,
                                                           const float *__restrict__ x, float *__restrict__ y, int S, int I, int O) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int o = blockIdx.x * 8 + warp, s0 = blockIdx.y * NS;
    pdl_trigger();
    pdl_wait();
    if (o >= O) return;
    const int rb = (I + 1) / 2, ng = (I + 31) / 32;
    const uint8_t *w = w4 + (size_t)o * rb;
    float acc[NS];
#pragma unroll
    for (int s = 0; s < NS; s++) acc[s] = 0.f;
    for (int g = 0; g < ng; g++) {
        const int e = g * 32 + lane;
        float wv = 0.f;
        if (e < I) { const uint8_t b = w[e >> 1]; wv = (float)((int)((e & 1) ? (b >> 4) : (b & 15)) - 8); }
        const float sc = scale[(size_t)o * ng + g];
#pragma unroll
        for (int s = 0; s < NS; s++) {
            float p = (e < I && s0 + s < S) ? __fmul_rn(x[(size_t)(s0 + s) * I + e], wv) : 0.f;
            for (int off = 16; off > 0; off >>= 1) p = __fadd_rn(p, __shfl_xor_sync(0xffffffffu, p, off));
            acc[s] = __fadd_rn(acc[s], __fmul_rn(p, sc));
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NS; s++) if (s0 + s < S) y[(size_t)(s0 + s) * O + o] = acc[s];
    }
}

int launch_i4g_f32_rows(const uint8_t *w4, const float *scale, const float *x, float *y, int S, int I, int O, cudaStream_t st) {
    if (S <= 0 || O <= 0) return 0;
    if (I <= 0) return moty_set_error(MOTY_CUDA_EARG, "i4g_f32: I=%d", I);
    const dim3 grid((O + 7) / 8, (S + 3) / 4);
    if (grid.y > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "i4g_f32: S=%d in one call", S);
    CK(moty_launch_pdl(i4g_f32_rows_kernel<4>, grid, dim3(256), (size_t)0, st, w4, scale, x, y, S, I, O));
    return 0;
}
