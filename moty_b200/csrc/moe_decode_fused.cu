// moe_decode_fused.cu -- one token through a routed int8 MoE layer in ONE launch.
//
// Replaces moe_d1_core (nn/moe.c:33-153) and the per-token body of OLMoE's moe()
// (engines/olmoe.c:219-244) including the router's softmax + top-K
// (runtime/moecache.c:97-111): the three kernels of moe_decode.cu (route, gate/up, down)
// cost three launch latencies for ~50 MB of weights; here
//   phase 0  warp 0 of every CTA routes the token (route_row_warp, redundantly: 64-128
//            logits) while the other warps take the maximum of x; then x -> int8
//            (moty_hw_qrow_i8, hw/hw_quant.h:9-16)
//   phase 1  gate and up rows of the K selected experts, silu(g)*u -> h[k][i] (global)
//   (the first down-projection weights of every warp are requested here: they depend
//    only on the routing, so they travel while the grid meets)
//   barrier  all CTAs are resident (cooperative launch); a counting barrier with a
//            BOUNDED spin: on expiry the CTA records an error and leaves
//   phase 2  h[k] -> int8 per expert (nn/moe.c:122), then for every output row d, in
//            selection order: out[d] = fma(w[k], ds[d]*sh[k]*dot(down_k[d], hq[k]), out[d])
// Operation for operation the arithmetic is that of moe_decode.cu and of the generic
// tile path, so the three produce identical bits.
#include "kernels.cuh"
#include "moe.cuh"
#include "route.cuh"
#include "gridbar.cuh"

namespace {

template <int N> struct LgF { static constexpr int v = 1 + LgF<N / 2>::v; };
template <> struct LgF<1> { static constexpr int v = 0; };

// N per-lane partial sums -> lane L holds the total of value (L >> (5 - log2 N))
template <int N>
__device__ __forceinline__ void reduce_multi_f(int (&v)[N], int lane) {
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

struct MoeFusedArgs {
    const float *logits; int E, norm_topk;
    int *idx_out; float *w_out;                   // [K], written by CTA 0 (the caller may read them afterwards)
    const int8_t *g, *u, *d; const float *gs, *us, *ds;
    size_t gstride, gsstride, dstride, dsstride;  // per expert, in elements
    const float *x; float *h; float *out;         // x [D], h [K][I] scratch, out [D]
    float *rows;                                  // optional [K][D]: every selected expert's own output row, zeros for experts
                                                  // that live on another GPU (the expert-parallel decode exchanges these)
    float *rows_peer[8]; int npeer;               // or: the [K][D] row tables of ALL ranks (peer memory, own table included):
                                                  // the rows of resident experts are stored straight into every table
    unsigned *bar;                                // [0] arrivals, [1] generation; arrivals are 0 between launches
    int *err;
    int K, I, D, e_lo, e_hi;
};

// LPRG: 128-bit loads per lane and gate/up row (D <= LPRG*512); LPRD: same for a down row (I <= LPRD*512);
// KB: experts of one down row in flight (KB * LPRD <= 16).
template <int LPRG, int LPRD, int KB>
__global__ void __launch_bounds__(256, 2) moe_dec_fused_kernel(MoeFusedArgs a) {
    extern __shared__ int4 smem4[];               // xq [D] in phase 1, hq [K][I] in phase 2; then E floats
    __shared__ float red[8];
    __shared__ float sx_s;
    __shared__ int idx_s[64];
    __shared__ float w_s[64];
    __shared__ float sh_s[64];
    __shared__ int loc_s[64];
    __shared__ int gave_up;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int D = a.D, D16 = D / 16, I = a.I, I16 = I / 16, K = a.K;
    const int nwarps = gridDim.x * 8, gw = blockIdx.x * 8 + warp;
    const size_t abytes = (size_t)K * I > (size_t)D ? (size_t)K * I : (size_t)D;
    float *p_s = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(smem4) + ((abytes + 15) & ~(size_t)15));

    // ---------------- phase 0: route || max |x|, then x -> int8 ----------------
    const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
    if (warp == 0) {
        route_row_warp(a.logits, a.E, K, p_s, 1, a.norm_topk, lane, idx_s, w_s, nullptr);
        if (lane == 0) { red[0] = 0.f; gave_up = 0; }
    } else {
        float amax = 0.f;
        for (int i = threadIdx.x - 32; i < D / 4; i += 224) {
            float4 v = x4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        amax = warp_max_f32(amax);
        if (lane == 0) red[warp] = amax;
    }
    __syncthreads();
    {
        float amax = red[0];
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
        if (threadIdx.x < K) loc_s[threadIdx.x] = idx_s[threadIdx.x] >= a.e_lo && idx_s[threadIdx.x] < a.e_hi;
        if (blockIdx.x == 0 && threadIdx.x < K) {
            a.idx_out[threadIdx.x] = idx_s[threadIdx.x];
            a.w_out[threadIdx.x] = w_s[threadIdx.x];
        }
    }
    __syncthreads();
    const float sx = sx_s;

    // ---------------- phase 1: gate / up rows, activation fused ----------------
    {
        constexpr int R = 2;
        const int nrg = (I + R - 1) / R, nunits = K * nrg;
        int4 wg[R][LPRG], wu[R][LPRG];
        float sc_g = 0.f, sc_u = 0.f;
        bool local = false;
        // after the reduction lane L reports value (L >> 3): 0,1 = gate rows, 2,3 = up rows
        const int my = lane >> 3, my_r = my & 1;
        auto issue = [&](int t) {
            const int k = t / nrg, rg = t - k * nrg;
            local = loc_s[k] != 0;
            if (!local) return;
            const size_t le = (size_t)(idx_s[k] - a.e_lo);
#pragma unroll
            for (int r = 0; r < R; r++) {
                int i = rg * R + r < I ? rg * R + r : I - 1;
                const int4 *pg = reinterpret_cast<const int4 *>(a.g + le * a.gstride) + (size_t)i * D16;
                const int4 *pu = reinterpret_cast<const int4 *>(a.u + le * a.gstride) + (size_t)i * D16;
#pragma unroll
                for (int j = 0; j < LPRG; j++) {
                    int kk = j * 32 + lane;
                    wg[r][j] = kk < D16 ? ldg_stream16(pg + kk) : make_int4(0, 0, 0, 0);
                    wu[r][j] = kk < D16 ? ldg_stream16(pu + kk) : make_int4(0, 0, 0, 0);
                }
            }
            int i = rg * R + my_r; i = i < I ? i : I - 1;
            sc_g = __ldg(a.gs + le * a.gsstride + i);
            sc_u = __ldg(a.us + le * a.gsstride + i);
        };
        int t0 = gw;
        if (t0 < nunits) issue(t0);
        while (t0 < nunits) {
            const int k = t0 / nrg, rg = t0 - k * nrg;
            const bool was_local = local;
            int flat[4] = {0, 0, 0, 0};
            if (was_local) {
#pragma unroll
                for (int j = 0; j < LPRG; j++) {
                    int kk = j * 32 + lane; kk = kk < D16 ? kk : D16 - 1;
                    int4 xv = smem4[kk];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        flat[r] = dp4a4(wg[r][j], xv, flat[r]);
                        flat[2 + r] = dp4a4(wu[r][j], xv, flat[2 + r]);
                    }
                }
            }
            reduce_multi_f<4>(flat, lane);
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

    // ---------------- down weights of this warp's first row: on their way during the barrier ----------------
    int4 wv[KB][LPRD];
    float scl[KB];
    auto issue_down = [&](int d, int k0) {
#pragma unroll
        for (int kb = 0; kb < KB; kb++) {
            const int k = k0 + kb;
            scl[kb] = 0.f;
#pragma unroll
            for (int j = 0; j < LPRD; j++) wv[kb][j] = make_int4(0, 0, 0, 0);
            if (k < K && loc_s[k]) {
                const size_t le = (size_t)(idx_s[k] - a.e_lo);
                const int4 *p = reinterpret_cast<const int4 *>(a.d + le * a.dstride) + (size_t)d * I16;
#pragma unroll
                for (int j = 0; j < LPRD; j++) {
                    int kk = j * 32 + lane;
                    if (kk < I16) wv[kb][j] = ldg_stream16(p + kk);
                }
                scl[kb] = __ldg(a.ds + le * a.dsstride + d);
            }
        }
    };
    if (gw < D) issue_down(gw, 0);

    // ---------------- grid barrier (bounded) ----------------
    if (!grid_barrier_bounded(a.bar, &gave_up)) {
        if (threadIdx.x == 0) atomicExch(a.err, 1);
        return;
    }

    // ---------------- phase 2: h -> int8 per expert, down rows, weighted sum in selection order ----------------
    if (K == 1) {
        // one row (a dense FFN run as a one-expert block): the whole CTA quantizes it, one L2 round trip per pass,
        // instead of one warp walking it alone
        const bool local = loc_s[0] != 0;
        const float4 *h4 = reinterpret_cast<const float4 *>(a.h);
        float amax = 0.f;
        if (local)
            for (int i = threadIdx.x; i < I / 4; i += 256) {
                float4 v = __ldcg(h4 + i);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        amax = warp_max_f32(amax);
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
        const float s = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, s);
        int *hq = reinterpret_cast<int *>(smem4);
        for (int i = threadIdx.x; i < I / 4; i += 256) {
            int word = 0;
            if (local) {
                float4 v = __ldcg(h4 + i);
                int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
                int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
                word = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
            }
            hq[i] = word;
        }
        if (threadIdx.x == 0) sh_s[0] = s;
    } else
    for (int k = warp; k < K; k += 8) {
        const bool local = loc_s[k] != 0;
        const float4 *h4 = reinterpret_cast<const float4 *>(a.h + (size_t)k * I);
        float amax = 0.f;
        if (local)
            for (int i = lane; i < I / 4; i += 32) {
                float4 v = __ldcg(h4 + i);
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        amax = warp_max_f32(amax);
        const float s = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, s);
        int *hq = reinterpret_cast<int *>(smem4) + (size_t)k * (I / 4);
        for (int i = lane; i < I / 4; i += 32) {
            int word = 0;
            if (local) {
                float4 v = __ldcg(h4 + i);
                int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
                int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
                word = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
            }
            hq[i] = word;
        }
        if (lane == 0) sh_s[k] = s;
    }
    __syncthreads();

    constexpr int SHD = 5 - LgF<KB>::v;               // lanes sharing one reduced value
    for (int d = gw; d < D; d += nwarps) {
        float acc = 0.f;
        for (int k0 = 0; k0 < K; k0 += KB) {
            if (d != gw || k0 != 0) issue_down(d, k0);
            int flat[KB];
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                flat[kb] = 0;
                const int k = k0 + kb < K ? k0 + kb : K - 1;
#pragma unroll
                for (int j = 0; j < LPRD; j++) {
                    int kk = j * 32 + lane; kk = kk < I16 ? kk : I16 - 1;
                    int4 hv = smem4[(size_t)k * I16 + kk];
                    flat[kb] = dp4a4(wv[kb][j], hv, flat[kb]);
                }
            }
            // the scale of value kb travels to the lane that reports it
            float myscl = 0.f;
#pragma unroll
            for (int kb = 0; kb < KB; kb++) if ((lane >> SHD) == kb) myscl = scl[kb];
            reduce_multi_f<KB>(flat, lane);
            const int mykb = lane >> SHD, myk = k0 + mykb;
            // ds[d] * sh[k] * dot, left to right (nn/moe.c:139)
            const float val = __fmul_rn(__fmul_rn(myscl, sh_s[myk < K ? myk : K - 1]), (float)flat[0]);
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                const int k = k0 + kb;
                const float v = __shfl_sync(0xffffffffu, val, kb << SHD);
                if (k < K && loc_s[k]) acc = fmaf(w_s[k], v, acc);        // out += w[k] * value (nn/moe.c:148)
                if (a.rows && lane == 0 && k < K) a.rows[(size_t)k * D + d] = loc_s[k] ? v : 0.f;
                if (a.npeer > 0 && lane < a.npeer && k < K && loc_s[k]) a.rows_peer[lane][(size_t)k * D + d] = v;   // one peer per lane
            }
        }
        if (lane == 0) a.out[d] = acc;
    }
}

template <int LPRG, int LPRD, int KB>
int launch_fused_t(const MoeFusedArgs &a, int sms, cudaStream_t st) {
    auto k = moe_dec_fused_kernel<LPRG, LPRD, KB>;
    size_t abytes = (size_t)a.K * a.I > (size_t)a.D ? (size_t)a.K * a.I : (size_t)a.D;
    size_t smem = ((abytes + 15) & ~(size_t)15) + (size_t)a.E * 4;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "moe_decode_fused: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    int per_sm = cached_per_sm[dev];
    if (per_sm < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "moe_decode_fused: kernel does not fit (smem %zu)", smem);
    int units = a.K * ((a.I + 1) / 2);
    if (units < a.D) units = a.D;
    int ctas = sms * per_sm;
    if (ctas > (units + 7) / 8) ctas = (units + 7) / 8;
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

}  // namespace

// Supports D, I multiples of 16, D <= 2048, I <= 4096, K <= 64, E <= 2048.
bool moe_decode_fused_q8_supported(int E, int K, int I, int D) {
    return E >= 1 && E <= 2048 && K >= 1 && K <= 64 && K <= E && I % 16 == 0 && D % 16 == 0 && D <= 2048 &&
           I <= 4096 && (size_t)K * I <= 160 * 1024;
}

// bar: two unsigned words, both zero before the first launch; err: set to 1 when a barrier wait expired.
int launch_moe_decode_fused_q8(const float *logits, int E, int norm_topk, int *idx_out, float *w_out,
                               const int8_t *g, const int8_t *u, const int8_t *d, const float *gs, const float *us,
                               const float *ds, size_t gstride, size_t gsstride, size_t dstride, size_t dsstride,
                               const float *x, float *h, float *out, float *rows, int K, int I, int D, int e_lo, int e_hi,
                               unsigned *bar, int *err, int sms, cudaStream_t st, float *const *rows_peer, int npeer) {
    if (!moe_decode_fused_q8_supported(E, K, I, D))
        return moty_set_error(MOTY_CUDA_EARG, "moe_decode_fused: E=%d K=%d I=%d D=%d", E, K, I, D);
    MoeFusedArgs a;
    a.logits = logits; a.E = E; a.norm_topk = norm_topk; a.idx_out = idx_out; a.w_out = w_out;
    a.g = g; a.u = u; a.d = d; a.gs = gs; a.us = us; a.ds = ds;
    a.gstride = gstride; a.gsstride = gsstride; a.dstride = dstride; a.dsstride = dsstride;
    a.x = x; a.h = h; a.out = out; a.rows = rows; a.npeer = npeer > 8 ? 0 : npeer;
    for (int r = 0; r < 8; r++) a.rows_peer[r] = rows_peer && r < npeer ? rows_peer[r] : nullptr;
    a.bar = bar; a.err = err; a.K = K; a.I = I; a.D = D; a.e_lo = e_lo; a.e_hi = e_hi;
    const int lprg = (D / 16 + 31) / 32, lprd = (I / 16 + 31) / 32;
    if (lprg <= 2) {
        if (lprd <= 2) return launch_fused_t<2, 2, 8>(a, sms, st);
        if (lprd <= 4) return launch_fused_t<2, 4, 4>(a, sms, st);
        return launch_fused_t<2, 8, 2>(a, sms, st);
    }
    if (lprd <= 2) return launch_fused_t<4, 2, 8>(a, sms, st);
    if (lprd <= 4) return launch_fused_t<4, 4, 4>(a, sms, st);
    return launch_fused_t<4, 8, 2>(a, sms, st);
}
