// moe_decode.cu -- one routed token through int8 experts in two streaming kernels.
//
// Replaces the S = 1 MoE block moe_d1_core (nn/moe.c:33-153) and the per-token body of
// OLMoE's moe() (engines/olmoe.c:219-244) after routing:
//   kernel A  x -> int8 once (moty_hw_qrow_i8), then for every selected expert k and
//             every FFN row i: g = gs[i]*sx*dot(gate_k[i], xq), u = us[i]*sx*dot(up_k[i], xq),
//             h[k][i] = silu(g) * u                      (nn/moe.c:95-121, hw/hw_ops.h:19-21)
//   kernel B  h[k] -> int8 per expert (nn/moe.c:122), then for every output row d, in
//             selection order k = 0..K-1: out[d] = fma(w[k], ds[d]*sh[k]*dot(down_k[d], hq[k]), out[d])
//             (nn/moe.c:132-149)
// Both stream the experts' weights exactly once with the same persistent round-robin
// scheme as the dense GEMV (gemv_q8_stream.cu); the arithmetic, operation for operation,
// is that of the generic path (tile kernels + act + combine), so the results are identical.
// Experts that are not resident on this GPU (expert-parallel shard) are skipped and
// contribute nothing to out.
#include "kernels.cuh"
#include "moe.cuh"
#include "route.cuh"

namespace {

template <int N>
__device__ __forceinline__ void reduce_multi_d(int (&v)[N], int lane) {
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

struct MoeDecArgs {
    const int *idx; const float *w;               // routing of the one token: [K]
    // kernel A may route the token itself (softmax gate; runtime/moecache.c:97-111): logits [E] -> every CTA's warp 0
    // forms the K selections in shared memory (redundantly: 64-128 logits) while the other warps take the maximum of x,
    // and CTA 0 leaves them in idx_out / w_out ( = idx / w) for kernel B.  logits == nullptr: idx / w were written by a
    // router launch before.
    const float *logits; int E, norm_topk; int *idx_out; float *w_out;
    const int8_t *g, *u, *d; const float *gs, *us, *ds;   // expert slabs (local experts only)
    size_t gstride, gsstride, dstride, dsstride;  // per expert, in elements
    const float *x; float *h; float *out;         // x [D], h [K][I] scratch, out [D]
    int K, I, D, e_lo, e_hi;
};

// ---- kernel A: gate and up rows of the K selected experts, activation fused ----
// unit = (k, pair of FFN rows); LPR 128-bit loads per lane and row (D <= LPR*512).
template <int LPR>
__global__ void __launch_bounds__(256, (LPR <= 2 ? 4 : 2)) moe_dec_gateup_kernel(MoeDecArgs a) {
    extern __shared__ int4 smem4[];
    __shared__ float red[8];
    __shared__ float sx_s;
    __shared__ int idx_s[64];
    __shared__ float w_s[64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int D = a.D, D16 = D / 16, I = a.I;
    constexpr int R = 2;
    const int nrg = (I + R - 1) / R, nunits = a.K * nrg;
    const int nwarps = gridDim.x * 8;
    const bool routing = a.logits != nullptr;

    int4 wg[R][LPR], wu[R][LPR];
    float sc_g = 0.f, sc_u = 0.f;
    bool local = false;
    // after the reduction lane L reports value (L >> 3): 0,1 = gate rows, 2,3 = up rows
    const int my = lane >> 3, my_r = my & 1;
    auto issue = [&](int t) {
        const int k = t / nrg, rg = t - k * nrg;
        const int e = routing ? idx_s[k] : a.idx[k];
        local = e >= a.e_lo && e < a.e_hi;
        if (!local) return;
        const size_t le = (size_t)(e - a.e_lo);
#pragma unroll
        for (int r = 0; r < R; r++) {
            int i = rg * R + r < I ? rg * R + r : I - 1;
            const int4 *pg = reinterpret_cast<const int4 *>(a.g + le * a.gstride) + (size_t)i * D16;
            const int4 *pu = reinterpret_cast<const int4 *>(a.u + le * a.gstride) + (size_t)i * D16;
#pragma unroll
            for (int j = 0; j < LPR; j++) {
                int kk = j * 32 + lane;
                wg[r][j] = kk < D16 ? ldg_stream16(pg + kk) : make_int4(0, 0, 0, 0);
                wu[r][j] = kk < D16 ? ldg_stream16(pu + kk) : make_int4(0, 0, 0, 0);
            }
        }
        int i = rg * R + my_r; i = i < I ? i : I - 1;
        sc_g = __ldg(a.gs + le * a.gsstride + i);
        sc_u = __ldg(a.us + le * a.gsstride + i);
    };
    int t0 = blockIdx.x * 8 + warp;
    pdl_trigger();
    pdl_wait();                                   // the logits (or the routing) and x come from earlier kernels
    if (!routing && t0 < nunits) issue(t0);

    // x -> int8 codes in shared memory (moty_hw_qrow_i8, hw/hw_quant.h:9-16); with routing inside, warp 0 routes meanwhile
    {
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
        float amax = 0.f;
        if (routing && warp == 0) {
            float *p_s = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(smem4) + (((size_t)D + 15) & ~(size_t)15));
            route_row_warp(a.logits, a.E, a.K, p_s, 1, a.norm_topk, lane, idx_s, w_s, nullptr);
        } else {
            const int first = routing ? threadIdx.x - 32 : threadIdx.x, step = routing ? 224 : 256;
            for (int i = first; i < D / 4; i += step) {
                float4 v = x4[i];
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
            amax = warp_max_f32(amax);
        }
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        if (routing) {
            if (t0 < nunits) issue(t0);
            if (blockIdx.x == 0 && threadIdx.x < a.K) { a.idx_out[threadIdx.x] = idx_s[threadIdx.x]; a.w_out[threadIdx.x] = w_s[threadIdx.x]; }
        }
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
        const float sx = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, sx);
        int *xq = reinterpret_cast<int *>(smem4);
        for (int i = threadIdx.x; i < D / 4; i += 256) {
            float4 v = x4[i];
            int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
            int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
            xq[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        if (threadIdx.x == 0) sx_s = sx;
    }
    __syncthreads();
    const float sx = sx_s;

    while (t0 < nunits) {
        const int k = t0 / nrg, rg = t0 - k * nrg;
        const bool was_local = local;
        int flat[4] = {0, 0, 0, 0};
        if (was_local) {
#pragma unroll
            for (int j = 0; j < LPR; j++) {
                int kk = j * 32 + lane; kk = kk < D16 ? kk : D16 - 1;
                int4 xv = smem4[kk];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    flat[r] = dp4a4(wg[r][j], xv, flat[r]);
                    flat[2 + r] = dp4a4(wu[r][j], xv, flat[2 + r]);
                }
            }
        }
        reduce_multi_d<4>(flat, lane);
        const float sg = sc_g, su = sc_u;
        t0 += nwarps;
        if (t0 < nunits) issue(t0);
        // the gate lane fetches the up sum of the same row from 16 lanes further
        const int upsum = __shfl_sync(0xffffffffu, flat[0], (lane + 16) & 31);
        const int i = rg * R + my_r;
        if (was_local && my < 2 && (lane & 7) == 0 && i < I) {
            // scale * sx * dot, left to right (nn/moe.c:107), then silu(g) * u (nn/moe.c:119)
            float gv = __fmul_rn(__fmul_rn(sg, sx), (float)flat[0]);
            float uv = __fmul_rn(__fmul_rn(su, sx), (float)upsum);
            a.h[(size_t)k * I + i] = moty_silu_mul(gv, uv);
        }
    }
}

// ---- kernel B: down rows of the K experts, weighted sum in selection order ----
// unit = pair of output rows d; for every k the two rows of down_k; KB experts in flight.
template <int LPR, int KB>
__global__ void __launch_bounds__(256, 2) moe_dec_down_kernel(MoeDecArgs a) {
    extern __shared__ int4 smem4[];               // hq [K][I] int8
    __shared__ float sh_s[64];
    __shared__ int loc_s[64];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int I = a.I, I16 = I / 16, D = a.D, K = a.K;
    constexpr int R = 2;
    const int nunits = (D + R - 1) / R, nwarps = gridDim.x * 8;

    pdl_trigger();
    pdl_wait();                                   // h comes from the kernel before this one
    // every warp quantizes the hidden rows of some experts: amax over the row, then the codes
    for (int k = warp; k < K; k += 8) {
        const int e = a.idx[k];
        const bool local = e >= a.e_lo && e < a.e_hi;
        const float4 *h4 = reinterpret_cast<const float4 *>(a.h + (size_t)k * I);
        float amax = 0.f;
        if (local)
            for (int i = lane; i < I / 4; i += 32) {
                float4 v = h4[i];
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        amax = warp_max_f32(amax);
        const float s = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, s);
        int *hq = reinterpret_cast<int *>(smem4) + (size_t)k * (I / 4);
        for (int i = lane; i < I / 4; i += 32) {
            int word = 0;
            if (local) {
                float4 v = h4[i];
                int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
                int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
                word = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
            }
            hq[i] = word;
        }
        if (lane == 0) { sh_s[k] = s; loc_s[k] = local; }
    }
    __syncthreads();

    const int my = lane >> 4;                     // after the reduction lane L reports row (L >> 4)
    for (int t = blockIdx.x * 8 + warp; t < nunits; t += nwarps) {
        const int d = t * R + my;
        const int dc = d < D ? d : D - 1;
        float acc = 0.f;
        for (int k0 = 0; k0 < K; k0 += KB) {
            int4 wv[KB][R][LPR];
            float scl[KB];
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                const int k = k0 + kb;
                scl[kb] = 0.f;
#pragma unroll
                for (int r = 0; r < R; r++)
#pragma unroll
                    for (int j = 0; j < LPR; j++) wv[kb][r][j] = make_int4(0, 0, 0, 0);
                if (k < K && loc_s[k]) {
                    const size_t le = (size_t)(a.idx[k] - a.e_lo);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        int row = t * R + r < D ? t * R + r : D - 1;
                        const int4 *p = reinterpret_cast<const int4 *>(a.d + le * a.dstride) + (size_t)row * I16;
#pragma unroll
                        for (int j = 0; j < LPR; j++) {
                            int kk = j * 32 + lane;
                            if (kk < I16) wv[kb][r][j] = ldg_stream16(p + kk);
                        }
                    }
                    scl[kb] = __ldg(a.ds + le * a.dsstride + dc);
                }
            }
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                const int k = k0 + kb;
                if (k >= K) break;
                int flat[R] = {0, 0};
#pragma unroll
                for (int j = 0; j < LPR; j++) {
                    int kk = j * 32 + lane; kk = kk < I16 ? kk : I16 - 1;
                    int4 hv = smem4[(size_t)k * I16 + kk];
#pragma unroll
                    for (int r = 0; r < R; r++) flat[r] = dp4a4(wv[kb][r][j], hv, flat[r]);
                }
                reduce_multi_d<R>(flat, lane);
                if (loc_s[k]) {
                    // ds[d] * sh[k] * dot, left to right (nn/moe.c:139), then out += w[k] * value (:148)
                    float val = __fmul_rn(__fmul_rn(scl[kb], sh_s[k]), (float)flat[0]);
                    acc = fmaf(__ldg(a.w + k), val, acc);
                }
            }
        }
        if ((lane & 15) == 0 && d < D) a.out[d] = acc;
    }
}

}  // namespace

// idx/w: routing of the token (device, [K]); h: scratch [K][I] f32.  Supports D, I multiples of 16,
// D <= 2048 and I <= 4096 (one K segment per row, all of a unit's loads in registers), K <= 64.
bool moe_decode_q8_supported(int K, int I, int D) {
    return K >= 1 && K <= 64 && I % 16 == 0 && D % 16 == 0 && D <= 2048 && I <= 4096 && (size_t)K * I <= 160 * 1024;
}

int launch_moe_decode_q8(const int *idx, const float *w, const int8_t *g, const int8_t *u, const int8_t *d,
                         const float *gs, const float *us, const float *ds, size_t gstride, size_t gsstride,
                         size_t dstride, size_t dsstride, const float *x, float *h, float *out,
                         int K, int I, int D, int e_lo, int e_hi, int sms, cudaStream_t st,
                         const float *logits, int E, int norm_topk) {
    if (!moe_decode_q8_supported(K, I, D)) return moty_set_error(MOTY_CUDA_EARG, "moe_decode: K=%d I=%d D=%d", K, I, D);
    if (logits && (E < K || E > 2048)) return moty_set_error(MOTY_CUDA_EARG, "moe_decode: routing inside wants K <= E <= 2048 (E=%d)", E);
    MoeDecArgs a;
    a.logits = logits; a.E = E; a.norm_topk = norm_topk; a.idx_out = const_cast<int *>(idx); a.w_out = const_cast<float *>(w);
    a.idx = idx; a.w = w; a.g = g; a.u = u; a.d = d; a.gs = gs; a.us = us; a.ds = ds;
    a.gstride = gstride; a.gsstride = gsstride; a.dstride = dstride; a.dsstride = dsstride;
    a.x = x; a.h = h; a.out = out; a.K = K; a.I = I; a.D = D; a.e_lo = e_lo; a.e_hi = e_hi;
    {
        int units = K * ((I + 1) / 2);
        int ctas = sms * 4; if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
        int lpr = (D / 16 + 31) / 32;
        size_t smem = logits ? (((size_t)D + 15) & ~(size_t)15) + (size_t)E * 4 : (size_t)D;
        if (lpr <= 2) CK(moty_launch_pdl(moe_dec_gateup_kernel<2>, dim3(ctas), dim3(256), smem, st, a));
        else CK(moty_launch_pdl(moe_dec_gateup_kernel<4>, dim3(ctas), dim3(256), smem, st, a));
    }
    {
        int units = (D + 1) / 2;
        int ctas = sms * 2; if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
        int lpr = (I / 16 + 31) / 32;
        size_t smem = (size_t)K * I;
        if (lpr <= 2) {
            auto k = moe_dec_down_kernel<2, 4>;
            if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
        } else if (lpr <= 4) {
            auto k = moe_dec_down_kernel<4, 2>;
            if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
        } else {
            auto k = moe_dec_down_kernel<8, 1>;
            if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
        }
    }
    return 0;
}
