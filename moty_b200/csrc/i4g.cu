// i4g.cu -- WF_I4G weights (grouped int4, group 32, f32 group scales, row-major nibbles) x
// row-quantized int8 activations: the integer path of moty_matmul_i4_grouped_s
// (nn/matmul.c:164-197 with IDOT4=1; kernel moty_hw_dot_i4g8p, hw/hw_quant.h:35-50 and
// hw/hw_avx512.h:155-176).
//
// Per (row, token) the reference forms, for every group of 32 weights, the exact integer
// d = sum((nibble - 8) * x) and adds ONE f32 term per group in ascending group order,
// acc = fma(scl[g], (float)d, acc) (its builds contract the multiply-add), and returns
// sx * acc.  The chain is sequential, so a lane owns a weight row and walks its groups in order;
// up to eight tokens ride along in registers.  A row's groups are 16 contiguous bytes each, the
// even element of a pair in the low nibble: the activation codes are split into even and odd
// elements once per CTA (shared memory, read by broadcast) so that four dp4a take the low
// nibbles and four the high ones; sum(nibble * x) - 8 * sum(x) gives d.
#include "kernels.cuh"

namespace {

struct I4GArgs {
    const uint8_t *w4; const float *scale;     // [O][I/2], [O][I/32]
    const int8_t *xi; const float *sx;         // row-quantized activations [S][I], [S]
    float *y;                                  // [S][O]
    int S, I, O;
};

constexpr int I4G_CH = 4;                      // groups per register chunk (two chunks alternate)

template <int NS>
__global__ void __launch_bounds__(256) i4g_rows_kernel(I4GArgs a) {
    extern __shared__ int4 smem_i4g[];
    const int I = a.I, ng = I / 32, O = a.O;
    int4 *xq_s = smem_i4g;                                              // [ng][NS][2]: even elements, odd elements
    int *x8_s = reinterpret_cast<int *>(smem_i4g + (size_t)ng * NS * 2);  // [ng][NS]: 8 * sum of the group's codes
    const int s0 = blockIdx.y * NS;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int o = blockIdx.x * 256 + warp * 32 + lane;
    const bool live = o < O;
    o = live ? o : O - 1;                                               // rows past the end: a valid row, nothing stored
    const uint4 *wr = reinterpret_cast<const uint4 *>(a.w4 + (size_t)o * (I / 2));
    const float *sr = a.scale + (size_t)o * ng;

    uint4 wA[I4G_CH], wB[I4G_CH]; float cA[I4G_CH], cB[I4G_CH];
    auto load = [&](uint4 (&wv)[I4G_CH], float (&cv)[I4G_CH], int g0) {
#pragma unroll
        for (int u = 0; u < I4G_CH; u++) {
            const int g = g0 + u < ng ? g0 + u : ng - 1;
            wv[u] = __ldg(wr + g); cv[u] = __ldg(sr + g);
        }
    };
    pdl_trigger();
    load(wA, cA, 0);                                                    // weights only: may overlap the previous kernel
    pdl_wait();                                                         // the codes come from the quantizer launch

    for (int i = threadIdx.x; i < ng * NS; i += 256) {
        const int g = i / NS, s = i - g * NS;
        int t = s0 + s; t = t < a.S ? t : a.S - 1;
        const int4 *src = reinterpret_cast<const int4 *>(a.xi + (size_t)t * I + (size_t)g * 32);
        const int4 x0 = src[0], x1 = src[1];
        int4 ev, od;
        ev.x = __byte_perm(x0.x, x0.y, 0x6420); od.x = __byte_perm(x0.x, x0.y, 0x7531);
        ev.y = __byte_perm(x0.z, x0.w, 0x6420); od.y = __byte_perm(x0.z, x0.w, 0x7531);
        ev.z = __byte_perm(x1.x, x1.y, 0x6420); od.z = __byte_perm(x1.x, x1.y, 0x7531);
        ev.w = __byte_perm(x1.z, x1.w, 0x6420); od.w = __byte_perm(x1.z, x1.w, 0x7531);
        xq_s[(size_t)i * 2] = ev; xq_s[(size_t)i * 2 + 1] = od;
        int sum = __dp4a(x0.x, 0x01010101, 0);
        sum = __dp4a(x0.y, 0x01010101, sum); sum = __dp4a(x0.z, 0x01010101, sum); sum = __dp4a(x0.w, 0x01010101, sum);
        sum = __dp4a(x1.x, 0x01010101, sum); sum = __dp4a(x1.y, 0x01010101, sum);
        sum = __dp4a(x1.z, 0x01010101, sum); sum = __dp4a(x1.w, 0x01010101, sum);
        x8_s[i] = 8 * sum;
    }
    __syncthreads();

    float acc[NS];
#pragma unroll
    for (int s = 0; s < NS; s++) acc[s] = 0.f;
    auto consume = [&](const uint4 (&wv)[I4G_CH], const float (&cv)[I4G_CH], int g0) {
#pragma unroll
        for (int u = 0; u < I4G_CH; u++) {
            const int g = g0 + u;
            if (g >= ng) break;
            const uint4 w = wv[u];
            const int l0 = w.x & 0x0f0f0f0f, l1 = w.y & 0x0f0f0f0f, l2 = w.z & 0x0f0f0f0f, l3 = w.w & 0x0f0f0f0f;
            const int h0 = (w.x >> 4) & 0x0f0f0f0f, h1 = (w.y >> 4) & 0x0f0f0f0f, h2 = (w.z >> 4) & 0x0f0f0f0f, h3 = (w.w >> 4) & 0x0f0f0f0f;
#pragma unroll
            for (int s = 0; s < NS; s++) {
                const int4 ev = xq_s[((size_t)g * NS + s) * 2], od = xq_s[((size_t)g * NS + s) * 2 + 1];
                int d = __dp4a(l0, ev.x, -x8_s[g * NS + s]);
                d = __dp4a(l1, ev.y, d); d = __dp4a(l2, ev.z, d); d = __dp4a(l3, ev.w, d);
                d = __dp4a(h0, od.x, d); d = __dp4a(h1, od.y, d); d = __dp4a(h2, od.z, d); d = __dp4a(h3, od.w, d);
                acc[s] = fmaf(cv[u], (float)d, acc[s]);                 // hw/hw_quant.h:47: acc += scl[g] * (float)d
            }
        }
    };
    for (int g0 = 0; g0 < ng; g0 += 2 * I4G_CH) {
        if (g0 + I4G_CH < ng) load(wB, cB, g0 + I4G_CH);
        consume(wA, cA, g0);
        if (g0 + 2 * I4G_CH < ng) load(wA, cA, g0 + 2 * I4G_CH);
        consume(wB, cB, g0 + I4G_CH);
    }
    if (!live) return;
#pragma unroll
    for (int s = 0; s < NS; s++)
        if (s0 + s < a.S) a.y[(size_t)(s0 + s) * O + o] = __fmul_rn(a.sx[s0 + s], acc[s]);   // nn/matmul.c:157: sx * dot
}

template <int NS>
int launch_i4g_t(const I4GArgs &a, cudaStream_t st) {
    const int ng = a.I / 32;
    const size_t smem = (size_t)ng * NS * 36;
    static size_t attr_smem[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "i4g: device %d", dev);
    if (smem > 48 * 1024 && smem > attr_smem[dev]) {
        CK(cudaFuncSetAttribute(i4g_rows_kernel<NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev] = smem;
    }
    dim3 grid((a.O + 255) / 256, (a.S + NS - 1) / NS);
    if (grid.y > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "i4g: S=%d in one call", a.S);
    CK(moty_launch_pdl(i4g_rows_kernel<NS>, grid, dim3(256), smem, st, a));
    return 0;
}

}  // namespace

// xi/sx: the S rows quantized per row (qrow_i8).  Group size 32, I a multiple of 32, I <= MOTY_QROW_MAX.
int launch_i4g_rows(const uint8_t *w4, const float *scale, const int8_t *xi, const float *sx, float *y,
                    int S, int I, int O, cudaStream_t st) {
    if (I % 32 != 0 || I <= 0 || I > MOTY_QROW_MAX || S <= 0 || O <= 0)
        return moty_set_error(MOTY_CUDA_EARG, "i4g: S=%d I=%d O=%d", S, I, O);
    I4GArgs a; a.w4 = w4; a.scale = scale; a.xi = xi; a.sx = sx; a.y = y; a.S = S; a.I = I; a.O = O;
    if (S > 4) return launch_i4g_t<8>(a, st);
    if (S > 2) return launch_i4g_t<4>(a, st);
    if (S == 2) return launch_i4g_t<2>(a, st);
    return launch_i4g_t<1>(a, st);
}

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
