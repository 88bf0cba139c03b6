// q4r4_gemv1.cu -- the Q4R4 decode GEMV for matrices with many rows (vocabulary, wide FFN):
// one activation row, one lane per weight row, no shuffles.
//
// Same arithmetic as q4r4_stream_kernel with GS = 1 (q4r4_stream.cu; moty_hw_q4r4_gemm_ref,
// hw/hw_q4r4.h:47-63: exact integer group sums, one fused multiply-add per group in ascending
// group order), restructured so that the instruction count per 64-byte group drops from ~96 to
// ~30 and the kernel is bound by HBM again instead of by issue slots:
//   * a warp unit is 8 consecutive 4-row blocks = 32 rows, lane = row; the lane walks its row in
//     chunks of PF groups whose loads are addressed by immediates off one pointer;
//   * two register buffers alternate: the next chunk (possibly the first of the warp's next
//     unit) is requested before the current one is consumed;
//   * the activation row is group-quantized by every CTA (moty_hw_quant_g32, hw/hw_q4r4.h:36-45)
//     into shared memory as codes plus one {scale, 8 * code sum} pair per group, read by broadcast.
#include "kernels.cuh"

namespace {

struct Q4G1Args {
    const uint8_t *w; const uint16_t *d;
    const float *x; float *y;
    int I, O;
};

__device__ __forceinline__ int dp4a_us1(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

template <int PF>
__global__ void __launch_bounds__(256, 2) q4r4_gemv1_kernel(Q4G1Args a) {
    extern __shared__ int4 sm4[];
    const int I = a.I, nb = I / 32, O = a.O;
    int8_t *xq_s = reinterpret_cast<int8_t *>(sm4);
    int2 *xr_s = reinterpret_cast<int2 *>(xq_s + I);                   // {scale bits, 8 * code sum} per group
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblk = (O + 3) / 4, nunits = (nblk + 7) / 8, nch = nb / PF;
    const int nwarps = gridDim.x * 8;
    int unit = blockIdx.x * 8 + warp, ci = 0;

    auto base_w = [&](int u) {
        int blk = u * 8 + (lane >> 2); blk = blk < nblk ? blk : nblk - 1;     // rows past the end: a valid block, nothing stored
        return a.w + (size_t)blk * nb * 64 + (lane & 3) * 16;
    };
    auto base_d = [&](int u) {
        int blk = u * 8 + (lane >> 2); blk = blk < nblk ? blk : nblk - 1;
        return a.d + (size_t)blk * nb * 4 + (lane & 3);
    };
    int4 wA[PF], wB[PF]; uint16_t dA[PF], dB[PF];
    auto load = [&](int4 (&wv)[PF], uint16_t (&dv)[PF], const uint8_t *wp, const uint16_t *dp) {
#pragma unroll
        for (int u = 0; u < PF; u++) { wv[u] = ldg_stream16(wp + u * 64); dv[u] = __ldg(dp + u * 4); }
    };
    const uint8_t *wp = base_w(unit); const uint16_t *dp = base_d(unit);
    pdl_trigger();
    if (unit < nunits) load(wA, dA, wp, dp);                            // weights only: may overlap the previous kernel
    pdl_wait();

    // ---- the activation row: one thread per group ----
    for (int g = threadIdx.x; g < nb; g += 256) {
        const float4 *xg4 = reinterpret_cast<const float4 *>(a.x + (size_t)g * 32);
        float4 v[8];
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = xg4[k];
        float amax = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++)
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w))));
        const float s = quant_scale(amax, 1e-30f);
        const float inv = __fdiv_rn(1.f, s);
        int tot = 0;
        int *dst = reinterpret_cast<int *>(xq_s + (size_t)g * 32);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            int c0 = quant_code(v[k].x, inv), c1 = quant_code(v[k].y, inv);
            int c2 = quant_code(v[k].z, inv), c3 = quant_code(v[k].w, inv);
            tot += c0 + c1 + c2 + c3;
            dst[k] = (c0 & 255) | ((c1 & 255) << 8) | ((c2 & 255) << 16) | ((c3 & 255) << 24);
        }
        xr_s[g] = make_int2(__float_as_int(s), 8 * tot);
    }
    __syncthreads();

    float acc = 0.f;
    // consume one chunk from (wv, dv) while the next one is requested into (wn, dn)
    auto chunk = [&](const int4 (&wv)[PF], const uint16_t (&dv)[PF], int4 (&wn)[PF], uint16_t (&dn)[PF]) {
        int n_unit = unit, n_ci = ci + 1;
        const uint8_t *n_wp = wp + PF * 64; const uint16_t *n_dp = dp + PF * 4;
        if (n_ci == nch) { n_ci = 0; n_unit = unit + nwarps; n_wp = base_w(n_unit); n_dp = base_d(n_unit); }
        if (n_unit < nunits) load(wn, dn, n_wp, n_dp);
        const int4 *xg = reinterpret_cast<const int4 *>(xq_s + (size_t)ci * PF * 32);
        const int2 *xr = xr_s + ci * PF;
#pragma unroll
        for (int u = 0; u < PF; u++) {
            const int4 w4 = wv[u];
            // low nibbles as they are; high nibbles stay in place (16 x their value) and are read as UNSIGNED
            // bytes by dp4a, the exact factor 16 is shifted out of the sum afterwards
            const int4 x0 = xg[2 * u], x1 = xg[2 * u + 1];
            int sraw = __dp4a(w4.x & 0x0f0f0f0f, x0.x, 0);
            sraw = __dp4a(w4.y & 0x0f0f0f0f, x0.y, sraw);
            sraw = __dp4a(w4.z & 0x0f0f0f0f, x0.z, sraw);
            sraw = __dp4a(w4.w & 0x0f0f0f0f, x0.w, sraw);
            int s16 = dp4a_us1((unsigned)w4.x & 0xf0f0f0f0u, x1.x, 0);
            s16 = dp4a_us1((unsigned)w4.y & 0xf0f0f0f0u, x1.y, s16);
            s16 = dp4a_us1((unsigned)w4.z & 0xf0f0f0f0u, x1.z, s16);
            s16 = dp4a_us1((unsigned)w4.w & 0xf0f0f0f0u, x1.w, s16);
            sraw += s16 >> 4;
            const int2 r = xr[u];
            // token-by-token formula (hw/hw_q4r4.h:58-59): (float)(sum - 8 * xsum) * (d * xs), one fma per group
            acc = fmaf((float)(sraw - r.y), __fmul_rn(f16bits_to_f32(dv[u]), __int_as_float(r.x)), acc);
        }
        if (ci == nch - 1) {                                            // the row is complete
            const int o = unit * 32 + lane;
            if (o < O) a.y[o] = acc;
            acc = 0.f;
        }
        unit = n_unit; ci = n_ci; wp = n_wp; dp = n_dp;
    };
    while (unit < nunits) {
        chunk(wA, dA, wB, dB);
        if (unit >= nunits) break;
        chunk(wB, dB, wA, dA);
    }
}

template <int PF>
int launch_g1_t(const Q4G1Args &a, int sms, cudaStream_t st) {
    const int nb = a.I / 32;
    size_t smem = (size_t)a.I + (size_t)nb * 8;
    auto k = q4r4_gemv1_kernel<PF>;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv1: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    int per_sm = cached_per_sm[dev];
    if (per_sm < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "q4r4_gemv1: kernel does not fit (smem %zu)", smem);
    const int nunits = (((a.O + 3) / 4) + 7) / 8;
    int ctas = sms * per_sm;
    if (ctas > (nunits + 7) / 8) ctas = (nunits + 7) / 8;
    CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
    return 0;
}

}  // namespace

// many rows, group count a multiple of 8, an aligned f32 row
bool q4r4_gemv1_supported(int I, int O, int sms) {
    return I % 256 == 0 && I > 0 && I <= MOTY_QROW_MAX && ((O + 3) / 4) / 8 >= sms * 12;
}

int launch_q4r4_gemv1(const uint8_t *w, const uint16_t *d, const float *x, float *y, int I, int O, int sms, cudaStream_t st) {
    if (!q4r4_gemv1_supported(I, O, sms)) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv1: I=%d O=%d", I, O);
    Q4G1Args a; a.w = w; a.d = d; a.x = x; a.y = y; a.I = I; a.O = O;
    return launch_g1_t<8>(a, sms, st);
}
