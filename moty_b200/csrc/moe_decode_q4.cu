// moe_decode_q4.cu -- one routed token through Q4R4 experts in two streaming kernels.
//
// No reference engine stores experts as Q4R4; the arithmetic is the composition the
// Qwen3-30B-A3B-shaped configuration is checked against: per selected expert the three
// projections of moty_matmul_q4r4_s with one token (token-by-token kernel,
// hw/hw_q4r4.h:47-63: offset removed in the integers, one fused multiply-add per group
// in ascending group order), SiLU * up between them (hw/hw_ops.h:19-21), group-of-32
// re-quantization of the hidden row (hw/hw_q4r4.h:36-45), and the weighted sum in
// selection order (nn/moe.c:146-149).  Operation for operation it is the generic path
// (q4r4_small_kernel tiles + act + combine), so results are bit-identical to it.
// The step layout and its helpers are in q4_decode.cuh.
#include "kernels.cuh"
#include "moe.cuh"
#include "q4_decode.cuh"

namespace {

struct MoeDec4Args {
    const int *idx; const float *w;
    const uint8_t *g, *u, *d; const uint16_t *gs, *us, *ds;    // expert slabs (local experts)
    size_t gstride, gsstride, dstride, dsstride;               // per expert, in elements
    const float *x; float *h; float *out;
    int K, I, D, e_lo, e_hi;
};

// ---- kernel A: gate and up blocks of the K selected experts, activation fused ----
__global__ void __launch_bounds__(256) moe_dec4_gateup_kernel(MoeDec4Args a) {
    extern __shared__ int4 sm4[];
    const int D = a.D, nb = D / 32, I = a.I;
    int8_t *xq_s = reinterpret_cast<int8_t *>(sm4);
    float *xs_s = reinterpret_cast<float *>(xq_s + D);
    int *xsum_s = reinterpret_cast<int *>(xs_s + nb);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gl = lane >> 2, r = lane & 3;
    const int prev = (lane + 28) & 31;
    const int nblk = (I + 3) / 4, nit = (nb + 7) / 8, nunits = a.K * nblk, nwarps = gridDim.x * 8;
    pdl_trigger();
    pdl_wait();                                                // the routing and x come from earlier kernels
    quant_groups(a.x, nb, xq_s, xs_s, xsum_s, threadIdx.x, 256);
    __syncthreads();
    for (int t = blockIdx.x * 8 + warp; t < nunits; t += nwarps) {
        const int k = t / nblk, ob = t - k * nblk;
        const int e = a.idx[k];
        if (e < a.e_lo || e >= a.e_hi) continue;               // warp-uniform
        const size_t le = (size_t)(e - a.e_lo);
        const uint8_t *gb = a.g + le * a.gstride + (size_t)ob * nb * 64, *ub = a.u + le * a.gstride + (size_t)ob * nb * 64;
        const uint16_t *gd = a.gs + le * a.gsstride + (size_t)ob * nb * 4, *ud = a.us + le * a.gsstride + (size_t)ob * nb * 4;
        float accg = 0.f, accu = 0.f;
        for (int it0 = 0; it0 < nit; it0 += 2) {               // two steps of gate and of up in flight
            int4 wgv[2], wuv[2]; uint16_t dgv[2], duv[2];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int g = (it0 + q) * 8 + gl;
                wgv[q] = wuv[q] = make_int4(0, 0, 0, 0); dgv[q] = duv[q] = 0;
                if (it0 + q < nit && g < nb) {
                    wgv[q] = ldg_stream16(gb + (size_t)(it0 + q) * 512 + lane * 16);
                    wuv[q] = ldg_stream16(ub + (size_t)(it0 + q) * 512 + lane * 16);
                    dgv[q] = __ldg(gd + (size_t)(it0 + q) * 32 + lane);
                    duv[q] = __ldg(ud + (size_t)(it0 + q) * 32 + lane);
                }
            }
#pragma unroll
            for (int q = 0; q < 2; q++) {
                if (it0 + q >= nit) break;
                const int g = (it0 + q) * 8 + gl;
                const bool valid = g < nb;
                const int gc = valid ? g : nb - 1;
                float fs, c0;
                q4_step_terms(wgv[q], dgv[q], xq_s, xs_s, xsum_s, gc, fs, c0);
                accg = q4_chain(accg, fs, c0, valid, gl, prev);
                q4_step_terms(wuv[q], duv[q], xq_s, xs_s, xsum_s, gc, fs, c0);
                accu = q4_chain(accu, fs, c0, valid, gl, prev);
            }
        }
        const int i = ob * 4 + r;
        if (gl == 7 && i < I) {
            a.h[(size_t)k * I + i] = moty_silu_mul(accg, accu);
        }
    }
}

// ---- kernel B: down blocks of the K experts, weighted sum in selection order ----
__global__ void __launch_bounds__(256) moe_dec4_down_kernel(MoeDec4Args a) {
    extern __shared__ int4 sm4[];
    const int I = a.I, nb = I / 32, D = a.D, K = a.K;
    int8_t *hq_s = reinterpret_cast<int8_t *>(sm4);                       // [K][I]
    float *hs_s = reinterpret_cast<float *>(hq_s + (size_t)K * I);        // [K][nb]
    int *hsum_s = reinterpret_cast<int *>(hs_s + (size_t)K * nb);         // [K][nb]
    __shared__ int loc_s[64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gl = lane >> 2, r = lane & 3;
    const int prev = (lane + 28) & 31;
    pdl_trigger();
    pdl_wait();                                                            // h comes from the kernel before this one
    if (threadIdx.x < K) { int e = a.idx[threadIdx.x]; loc_s[threadIdx.x] = e >= a.e_lo && e < a.e_hi; }
    __syncthreads();
    // hidden rows of the resident experts -> group-quantized codes (rows of absent experts are never read)
    for (int k = 0; k < K; k++)
        if (loc_s[k])
            quant_groups(a.h + (size_t)k * I, nb, hq_s + (size_t)k * I, hs_s + (size_t)k * nb, hsum_s + (size_t)k * nb,
                         threadIdx.x, 256);
    __syncthreads();
    const int nblk = (D + 3) / 4, nit = (nb + 7) / 8, nwarps = gridDim.x * 8;
    for (int ob = blockIdx.x * 8 + warp; ob < nblk; ob += nwarps) {
        float out = 0.f;
        for (int k = 0; k < K; k++) {
            if (!loc_s[k]) continue;                                       // warp-uniform
            const size_t le = (size_t)(a.idx[k] - a.e_lo);
            const uint8_t *wb = a.d + le * a.dstride + (size_t)ob * nb * 64;
            const uint16_t *db = a.ds + le * a.dsstride + (size_t)ob * nb * 4;
            float acc = 0.f;
            for (int it0 = 0; it0 < nit; it0 += 4) {
                int4 wv[4]; uint16_t dv[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int g = (it0 + q) * 8 + gl;
                    wv[q] = make_int4(0, 0, 0, 0); dv[q] = 0;
                    if (it0 + q < nit && g < nb) {
                        wv[q] = ldg_stream16(wb + (size_t)(it0 + q) * 512 + lane * 16);
                        dv[q] = __ldg(db + (size_t)(it0 + q) * 32 + lane);
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    if (it0 + q >= nit) break;
                    const int g = (it0 + q) * 8 + gl;
                    const bool valid = g < nb;
                    const int gc = valid ? g : nb - 1;
                    float fs, c0;
                    q4_step_terms(wv[q], dv[q], hq_s + (size_t)k * I, hs_s + (size_t)k * nb, hsum_s + (size_t)k * nb, gc, fs, c0);
                    acc = q4_chain(acc, fs, c0, valid, gl, prev);
                }
            }
            out = fmaf(__ldg(a.w + k), acc, out);                          // meaningful in the lanes of the last group
        }
        const int d = ob * 4 + r;
        if (gl == 7 && d < D) a.out[d] = out;
    }
}

}  // namespace

bool moe_decode_q4_supported(int K, int I, int D) {
    return K >= 1 && K <= 64 && I % 32 == 0 && D % 32 == 0 && D <= 8192 &&
           (size_t)K * I + (size_t)K * (I / 32) * 8 <= 160 * 1024;
}

int launch_moe_decode_q4(const int *idx, const float *w, const uint8_t *g, const uint8_t *u, const uint8_t *d,
                         const uint16_t *gs, const uint16_t *us, const uint16_t *ds, size_t gstride, size_t gsstride,
                         size_t dstride, size_t dsstride, const float *x, float *h, float *out,
                         int K, int I, int D, int e_lo, int e_hi, int sms, cudaStream_t st) {
    if (!moe_decode_q4_supported(K, I, D)) return moty_set_error(MOTY_CUDA_EARG, "moe_decode_q4: K=%d I=%d D=%d", K, I, D);
    MoeDec4Args a;
    a.idx = idx; a.w = w; a.g = g; a.u = u; a.d = d; a.gs = gs; a.us = us; a.ds = ds;
    a.gstride = gstride; a.gsstride = gsstride; a.dstride = dstride; a.dsstride = dsstride;
    a.x = x; a.h = h; a.out = out; a.K = K; a.I = I; a.D = D; a.e_lo = e_lo; a.e_hi = e_hi;
    {
        int units = K * ((I + 3) / 4);
        int ctas = sms * 4; if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
        size_t smem = (size_t)D + (size_t)(D / 32) * 8;
        CK(moty_launch_pdl(moe_dec4_gateup_kernel, dim3(ctas), dim3(256), smem, st, a));
    }
    {
        int units = (D + 3) / 4;
        int ctas = sms * 4; if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
        size_t smem = (size_t)K * I + (size_t)K * (I / 32) * 8;
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(moe_dec4_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(moty_launch_pdl(moe_dec4_down_kernel, dim3(ctas), dim3(256), smem, st, a));
    }
    return 0;
}
