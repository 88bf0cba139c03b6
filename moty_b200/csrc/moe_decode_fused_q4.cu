// moe_decode_fused_q4.cu -- one token through a routed Q4R4 MoE layer in ONE launch.
//
// Same plan as moe_decode_fused.cu (router in every CTA, gate/up, a bounded grid barrier,
// down) for experts stored as Q4R4 blocks; the arithmetic is that of moe_decode_q4.cu
// (token-by-token kernel hw/hw_q4r4.h:47-63 per projection, SiLU * up hw/hw_ops.h:19-21,
// group-of-32 re-quantization hw/hw_q4r4.h:36-45, weighted sum in selection order
// nn/moe.c:146-149), so the results are bit-identical to it and to the tile path.
//
//   phase 0  warp 0 routes the token; the other warps group-quantize x into shared memory
//   phase 1  a CTA takes (expert k, 32 consecutive FFN rows): each warp one 4-row block of
//            gate and of up (8 groups side by side, the chain hops by shuffle), all of a
//            block's codes requested at once; the 32 values silu(g)*u are exactly one
//            quantization group of the hidden row, so the CTA quantizes it on the spot and
//            writes 32 codes, a scale and a code sum: the f32 hidden row never exists
//   barrier  bounded (gridbar.cuh); the first down codes of every warp travel meanwhile
//   phase 2  the hidden codes (a few KB) into shared memory; a warp takes one 4-row block of
//            the down projection for ALL experts at once: lane = (expert, row) owns the whole
//            chain of its row (no shuffles), then the K row sums are added in selection order
#include "kernels.cuh"
#include "moe.cuh"
#include "route.cuh"
#include "q4_decode.cuh"
#include "gridbar.cuh"

namespace {

struct MoeFused4Args {
    const float *logits; int E, norm_topk;
    int *idx_out; float *w_out;
    const uint8_t *g, *u, *d; const uint16_t *gs, *us, *ds;
    size_t gstride, gsstride, dstride, dsstride;               // per expert, in elements
    const float *x; float *out;                                // x [D], out [D]
    float *rows;                                               // optional [K][D]: each selected expert's own output row (zeros if not resident)
    float *rows_peer[8]; int npeer;                            // or: all ranks' [K][D] row tables (peer memory): resident experts' rows go to every table
    int8_t *hq; float *hs; int *hsum;                          // hidden row, quantized: [K][I], [K][I/32], [K][I/32]
    unsigned *bar; int *err;
    int K, I, D, e_lo, e_hi;
};

constexpr int CH1 = 8;                                         // gate/up steps in flight per warp (x2 matrices)
constexpr int CHD = 12;                                        // down groups in flight per lane

// PHASE 0: the whole layer in one cooperative launch.  PHASE 1 / PHASE 2: the same code as two launches chained by
// programmatic dependent launch, split where the grid barrier stands -- the first leaves the hidden codes and the routing
// in global memory, the second picks the routing up from there (a cooperative launch cannot overlap its launch, or its
// successor's, with its neighbours; chained launches can).
template <int PHASE>
__global__ void __launch_bounds__(256, 2) moe_dec4_fused_kernel(MoeFused4Args a) {
    extern __shared__ int4 sm4[];
    __shared__ int idx_s[64];
    __shared__ float w_s[64];
    __shared__ int loc_s[64];
    __shared__ float hrow_s[32];
    __shared__ int gave_up;
    const int D = a.D, nbD = D / 32, I = a.I, nbI = I / 32, K = a.K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // phase 1 view of shared memory: x codes, scales, sums; phase 2 view: hidden codes (rows padded by 16
    // bytes so that the eight experts of a warp read different banks), scales and sums (odd row stride);
    // behind both: E floats for the router
    const int hstride = I + 16, nbs = nbI | 1;
    const size_t a1 = (size_t)D + (size_t)nbD * 8, a2 = (size_t)K * hstride + (size_t)K * nbs * 8;
    const size_t abytes = ((a1 > a2 ? a1 : a2) + 15) & ~(size_t)15;
    int8_t *xq_s = reinterpret_cast<int8_t *>(sm4);
    float *xs_s = reinterpret_cast<float *>(xq_s + D);
    int *xsum_s = reinterpret_cast<int *>(xs_s + nbD);
    int8_t *hq_s = reinterpret_cast<int8_t *>(sm4);
    float *hs_s = reinterpret_cast<float *>(hq_s + (size_t)K * hstride);
    int *hsum_s = reinterpret_cast<int *>(hs_s + (size_t)K * nbs);
    float *p_s = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(sm4) + abytes);

    if (PHASE != 0) { pdl_trigger(); pdl_wait(); }                    // logits / x (PHASE 1), hidden codes and routing (PHASE 2)
    if (PHASE == 2) {
        for (int k = threadIdx.x; k < K; k += 256) {
            const int e = a.idx_out[k];
            idx_s[k] = e; w_s[k] = a.w_out[k]; loc_s[k] = e >= a.e_lo && e < a.e_hi;
        }
        if (threadIdx.x == 0) gave_up = 0;
    } else
    // ---------------- phase 0: route || x -> group-quantized codes ----------------
    if (warp == 0) {
        route_row_warp(a.logits, a.E, K, p_s, 1, a.norm_topk, lane, idx_s, w_s, nullptr);
        __syncwarp();
        for (int k = lane; k < K; k += 32) {
            const int e = idx_s[k];
            loc_s[k] = e >= a.e_lo && e < a.e_hi;
            if (blockIdx.x == 0) { a.idx_out[k] = e; a.w_out[k] = w_s[k]; }
        }
        if (lane == 0) gave_up = 0;
    } else {
        quant_groups(a.x, nbD, xq_s, xs_s, xsum_s, threadIdx.x - 32, 224);
    }
    __syncthreads();

    // ---------------- phase 1: (expert, 32 FFN rows) per CTA; the hidden group is quantized on the spot ----------------
    if (PHASE != 2) {
        const int gl = lane >> 2, r = lane & 3, prev = (lane + 28) & 31;
        const int nit = (nbD + 7) / 8;
        for (int cu = blockIdx.x; cu < K * nbI; cu += gridDim.x) {
            const int k = cu / nbI, grp = cu - k * nbI;
            if (!loc_s[k]) continue;                                       // CTA-uniform
            const int ob = grp * 8 + warp;
            const size_t le = (size_t)(idx_s[k] - a.e_lo);
            const uint8_t *gb = a.g + le * a.gstride + (size_t)ob * nbD * 64, *ub = a.u + le * a.gstride + (size_t)ob * nbD * 64;
            const uint16_t *gd = a.gs + le * a.gsstride + (size_t)ob * nbD * 4, *ud = a.us + le * a.gsstride + (size_t)ob * nbD * 4;
            float accg = 0.f, accu = 0.f;
            for (int it0 = 0; it0 < nit; it0 += CH1) {
                int4 wgv[CH1], wuv[CH1]; uint16_t dgv[CH1], duv[CH1];
#pragma unroll
                for (int q = 0; q < CH1; q++) {
                    const int g = (it0 + q) * 8 + gl;
                    wgv[q] = wuv[q] = make_int4(0, 0, 0, 0); dgv[q] = duv[q] = 0;
                    if (it0 + q < nit && g < nbD) {
                        wgv[q] = ldg_stream16(gb + (size_t)(it0 + q) * 512 + lane * 16);
                        wuv[q] = ldg_stream16(ub + (size_t)(it0 + q) * 512 + lane * 16);
                        dgv[q] = __ldg(gd + (size_t)(it0 + q) * 32 + lane);
                        duv[q] = __ldg(ud + (size_t)(it0 + q) * 32 + lane);
                    }
                }
#pragma unroll
                for (int q = 0; q < CH1; q++) {
                    if (it0 + q >= nit) break;
                    const int g = (it0 + q) * 8 + gl;
                    const bool valid = g < nbD;
                    const int gc = valid ? g : nbD - 1;
                    float fs, c0;
                    q4_step_terms(wgv[q], dgv[q], xq_s, xs_s, xsum_s, gc, fs, c0);
                    accg = q4_chain(accg, fs, c0, valid, gl, prev);
                    q4_step_terms(wuv[q], duv[q], xq_s, xs_s, xsum_s, gc, fs, c0);
                    accu = q4_chain(accu, fs, c0, valid, gl, prev);
                }
            }
            if (gl == 7) {
                hrow_s[warp * 4 + r] = moty_silu_mul(accg, accu);
            }
            __syncthreads();
            if (warp == 0) {                                               // one quantization group (hw/hw_q4r4.h:36-45)
                const float v = hrow_s[lane];
                const float s = quant_scale(warp_max_f32(fabsf(v)), 1e-30f);
                const int c = quant_code(v, __fdiv_rn(1.f, s));
                const int tot = warp_sum_i32(c);
                a.hq[(size_t)k * I + grp * 32 + lane] = (int8_t)c;
                if (lane == 0) { a.hs[k * nbI + grp] = s; a.hsum[k * nbI + grp] = tot; }
            }
            __syncthreads();
        }
    }

    if (PHASE == 1) return;

    // ---------------- down: lane = (expert, row) of a 4-row block; first groups requested before the barrier ----------------
    const int kq = lane >> 2, r = lane & 3;
    const int nblkD = D / 4;
    int4 wd[CHD]; uint16_t dd[CHD];
    auto issue_down = [&](int ob, int k, int g0) {
#pragma unroll
        for (int q = 0; q < CHD; q++) { wd[q] = make_int4(0, 0, 0, 0); dd[q] = 0; }
        if (k >= K || !loc_s[k]) return;
        const size_t le = (size_t)(idx_s[k] - a.e_lo);
        const uint8_t *wb = a.d + le * a.dstride + (size_t)ob * nbI * 64 + r * 16;
        const uint16_t *db = a.ds + le * a.dsstride + (size_t)ob * nbI * 4 + r;
#pragma unroll
        for (int q = 0; q < CHD; q++)
            if (g0 + q < nbI) {
                wd[q] = ldg_stream16(wb + (size_t)(g0 + q) * 64);
                dd[q] = __ldg(db + (size_t)(g0 + q) * 4);
            }
    };
    // blocks are dealt warp-major so that they spread over all SMs: unit u <-> (warp, CTA)
    const int nslots = gridDim.x * 8, slot = warp * gridDim.x + blockIdx.x;
    if (slot < nblkD) issue_down(slot, kq, 0);

    if (PHASE == 0 && !grid_barrier_bounded(a.bar, &gave_up)) {
        if (threadIdx.x == 0) atomicExch(a.err, 1);
        return;
    }

    // ---------------- phase 2: hidden codes into shared memory, then the down blocks ----------------
    {
        const int I16 = I / 16;
        for (int i = threadIdx.x; i < K * I16; i += 256) {
            const int k = i / I16, j = i - k * I16;
            if (loc_s[k])
                *reinterpret_cast<int4 *>(hq_s + (size_t)k * hstride + j * 16) = __ldcg(reinterpret_cast<const int4 *>(a.hq) + i);
        }
        for (int i = threadIdx.x; i < K * nbI; i += 256) {
            const int k = i / nbI, g = i - k * nbI;
            if (loc_s[k]) { hs_s[k * nbs + g] = __ldcg(a.hs + i); hsum_s[k * nbs + g] = __ldcg(a.hsum + i); }
        }
    }
    __syncthreads();

    for (int ob = slot; ob < nblkD; ob += nslots) {
        float out = 0.f;
        for (int k0 = 0; k0 < K; k0 += 8) {                                // eight experts side by side
            const int k = k0 + kq;
            const bool active = k < K && loc_s[k < K ? k : 0];
            float acc = 0.f;
            for (int g0 = 0; g0 < nbI; g0 += CHD) {
                if (ob != slot || k0 != 0 || g0 != 0) issue_down(ob, k, g0);
                if (active) {
#pragma unroll
                    for (int q = 0; q < CHD; q++) {
                        if (g0 + q < nbI) {
                            float fs, c0;
                            q4_step_terms(wd[q], dd[q], hq_s + (size_t)k * hstride, hs_s + k * nbs, hsum_s + k * nbs, g0 + q, fs, c0);
                            acc = fmaf(fs, c0, acc);                       // ascending group order (hw/hw_q4r4.h:58-59)
                        }
                    }
                }
            }
#pragma unroll
            for (int kk = 0; kk < 8; kk++) {
                const float v = __shfl_sync(0xffffffffu, acc, kk * 4 + r);
                if (k0 + kk < K && loc_s[k0 + kk < K ? k0 + kk : 0]) out = fmaf(w_s[k0 + kk], v, out);   // nn/moe.c:148
                if (a.rows && kq == 0 && k0 + kk < K) a.rows[(size_t)(k0 + kk) * D + ob * 4 + r] = loc_s[k0 + kk] ? v : 0.f;
                if (kq < a.npeer && k0 + kk < K && loc_s[k0 + kk]) a.rows_peer[kq][(size_t)(k0 + kk) * D + ob * 4 + r] = v;   // lane group kq serves peer kq
            }
        }
        if (kq == 0) a.out[ob * 4 + r] = out;
    }
}

}  // namespace

bool moe_decode_fused_q4_supported(int E, int K, int I, int D) {
    if (!(E >= 1 && E <= 2048 && K >= 1 && K <= 64 && K <= E && I % 32 == 0 && D % 32 == 0 && I > 0 && D > 0)) return false;
    size_t a1 = (size_t)D + (size_t)(D / 32) * 8, a2 = (size_t)K * (I + 16) + (size_t)K * ((I / 32) | 1) * 8;
    return (a1 > a2 ? a1 : a2) + (size_t)E * 4 + 16 <= 96 * 1024;
}

// hq/hs/hsum: scratch for the quantized hidden rows ([K][I] bytes, [K][I/32] floats, [K][I/32] ints);
// bar: two zeroed words; err: set to 1 when the barrier wait expired.
int launch_moe_decode_fused_q4(const float *logits, int E, int norm_topk, int *idx_out, float *w_out,
                               const uint8_t *g, const uint8_t *u, const uint8_t *d, const uint16_t *gs,
                               const uint16_t *us, const uint16_t *ds, size_t gstride, size_t gsstride,
                               size_t dstride, size_t dsstride, const float *x, int8_t *hq, float *hs, int *hsum,
                               float *out, float *rows, int K, int I, int D, int e_lo, int e_hi, unsigned *bar, int *err,
                               int sms, cudaStream_t st, float *const *rows_peer, int npeer, int chained) {
    if (!moe_decode_fused_q4_supported(E, K, I, D))
        return moty_set_error(MOTY_CUDA_EARG, "moe_decode_fused_q4: E=%d K=%d I=%d D=%d", E, K, I, D);
    MoeFused4Args a;
    a.logits = logits; a.E = E; a.norm_topk = norm_topk; a.idx_out = idx_out; a.w_out = w_out;
    a.g = g; a.u = u; a.d = d; a.gs = gs; a.us = us; a.ds = ds;
    a.gstride = gstride; a.gsstride = gsstride; a.dstride = dstride; a.dsstride = dsstride;
    a.x = x; a.out = out; a.rows = rows; a.npeer = npeer > 8 ? 0 : npeer;
    for (int r = 0; r < 8; r++) a.rows_peer[r] = rows_peer && r < npeer ? rows_peer[r] : nullptr;
    a.hq = hq; a.hs = hs; a.hsum = hsum; a.bar = bar; a.err = err;
    a.K = K; a.I = I; a.D = D; a.e_lo = e_lo; a.e_hi = e_hi;
    size_t a1 = (size_t)D + (size_t)(D / 32) * 8, a2 = (size_t)K * (I + 16) + (size_t)K * ((I / 32) | 1) * 8;
    size_t smem = (((a1 > a2 ? a1 : a2) + 15) & ~(size_t)15) + (size_t)E * 4;
    auto k = moe_dec4_fused_kernel<0>;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "moe_decode_fused_q4: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {
        if (smem > 48 * 1024) {
            CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CK(cudaFuncSetAttribute(moe_dec4_fused_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CK(cudaFuncSetAttribute(moe_dec4_fused_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        }
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    int per_sm = cached_per_sm[dev];
    if (per_sm < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "moe_decode_fused_q4: kernel does not fit (smem %zu)", smem);
    int units = K * (I / 32), units2 = (D / 4 + 7) / 8;
    if (units < units2) units = units2;
    int ctas = sms * per_sm;
    if (ctas > units) ctas = units;
    if (chained) {                                             // the same grid twice: the down blocks are dealt over it warp-major
        CK(moty_launch_pdl(moe_dec4_fused_kernel<1>, dim3(ctas), dim3(256), smem, st, a));
        CK(moty_launch_pdl(moe_dec4_fused_kernel<2>, dim3(ctas), dim3(256), smem, st, a));
        return 0;
    }
    // cooperative: every CTA is resident before any runs, which the grid barrier relies on
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    CK(cudaLaunchKernelEx(&cfg, k, a));
    return 0;
}
