// attn.cu -- the attention core between the projections: QK-norm + RoPE, KV store, causal
// scores, softmax, accumulation (attn_tail, nn/attn.c:29-74, without q/k/v/o projections and
// without the optional output gate).  One layer's KV cache lives on the device, f32 or int8 rows
// with one scale per (head, position).
//
// This is f32 arithmetic whose summation order differs between the reference's own CPU tiers
// (hw/hw_ops.h:53-59 scalar, :168-199 NEON) and that calls libm (powf, cosf, sinf, expf): parity
// is by tolerance, not by bits.  The statements follow the scalar definitions; sums that the
// reference takes sequentially are taken by warps and combined.
#include "kernels.cuh"

namespace {

struct AttnArgs {
    float *q, *k; const float *v;        // [S][H*hd], [S][KV*hd], [S][KV*hd]; q and k are normed and rotated in place
    float *ctx;                          // [S][H*hd]
    const float *qn, *kn;                // per head dimension, or null
    float *K, *V;                        // f32 cache [KV][max_t][hd], or null
    int8_t *K8, *V8; float *Ks, *Vs;     // int8 cache [KV][max_t][hd] + scales [KV][max_t], or null
    int S, pos_base, H, KV, hd, rot, max_t;
    float theta, eps, scale;
    // gemma's attention (engines/gemma.c:299-386): p-RoPE on pairs (j, j + hd/2) with rot = rotated pairs and frequency
    // theta^(-2j/hd); a value norm with gains vn; on sliding layers only the last `window` positions (0 = all)
    int gemma, window; const float *vn;
    int *err;                            // device word set when *pos_dev is outside [0, pos_base]
    const int *pos_dev;                  // when set, the first position is read from the device (a captured decode step
                                         // is replayed with a position that moves); pos_base then only sizes the launch
};

__device__ __forceinline__ double block_sum_f64(double v, double *red) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double s = 0;
    for (int i = 0; i < nw; i++) s += red[i];
    return s;
}
__device__ __forceinline__ float block_max_f32(float v, float *red) {
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float m = red[0];
    for (int i = 1; i < nw; i++) m = fmaxf(m, red[i]);
    return m;
}
__device__ __forceinline__ float block_sum_f32(float v, float *red) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; i++) s += red[i];
    return s;
}

// One CTA per (token, head slot): slots 0..H-1 are query heads, H..H+KV-1 key/value heads.
// Thread i owns dimension i of the head (blockDim >= hd).
__global__ void __launch_bounds__(256) attn_prep_kernel(AttnArgs a) {
    __shared__ double red64[8];
    __shared__ float red32[8];
    __shared__ float xs[256];
    const int s = blockIdx.x, slot = blockIdx.y, i = threadIdx.x, hd = a.hd;
    pdl_trigger();
    pdl_wait();                                                // q, k, v come from the projections before this launch
    const bool isq = slot < a.H;
    const int hh = isq ? slot : slot - a.H;
    float *row = isq ? a.q + (size_t)s * a.H * hd + (size_t)hh * hd : a.k + (size_t)s * a.KV * hd + (size_t)hh * hd;
    const float *nw = isq ? a.qn : a.kn;
    int p0 = a.pos_base;
    if (a.pos_dev) {
        // the device counter may not leave [0, pos_base] (pos_base is the documented maximum and sized the cache check on
        // the host): a stale or over-replayed counter is clamped instead of storing past the cache, and reported
        p0 = *a.pos_dev;
        if (p0 < 0 || p0 > a.pos_base) { if (i == 0 && a.err) atomicExch(a.err, 1); p0 = p0 < 0 ? 0 : a.pos_base; }
    }
    const int pos = p0 + s;
    float x = i < hd ? row[i] : 0.f;
    if (nw) {                                                  // hw/hw_ops.h:14-18
        const double ms = block_sum_f64((double)x * (double)x, red64);
        const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / hd), a.eps)));
        if (i < hd) x = __fmul_rn(__fmul_rn(x, r), nw[i]);
    }
    if (i < hd) xs[i] = x;
    __syncthreads();
    // nn/rope.c:39-49: pairs (j, j + rot/2), angle = pos / theta^(2j/rot); gemma (engines/gemma.c:287-297): pairs
    // (j, j + hd/2) for j < rot, angle = pos * theta^(-2j/hd)
    const int half = a.gemma ? hd / 2 : a.rot / 2, nang = a.gemma ? a.rot : a.rot / 2;
    if (i < 2 * half) {
        const int j = i < half ? i : i - half;
        if (j < nang) {
            const float angle = a.gemma ? __fmul_rn((float)pos, powf(a.theta, __fdiv_rn(__fmul_rn(-2.0f, (float)j), (float)hd)))
                                        : __fdiv_rn((float)pos, powf(a.theta, __fdiv_rn((float)(2 * j), (float)a.rot)));
            const float c = cosf(angle), sn = sinf(angle);
            const float lo = xs[j], hi = xs[j + half];
            x = i < half ? __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn)) : __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
        }
    }
    if (i < hd) row[i] = x;
    if (isq) return;
    // KV store (nn/attn.c:49-60)
    const size_t slotp = (size_t)hh * a.max_t + pos;
    float vv = i < hd ? a.v[(size_t)s * a.KV * hd + (size_t)hh * hd + i] : 0.f;
    if (a.vn) {                                                // gemma's value norm (engines/gemma.c:320-324): same norm, gains vn
        const double ms = block_sum_f64((double)vv * (double)vv, red64);
        const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / hd), a.eps)));
        if (i < hd) vv = __fmul_rn(__fmul_rn(vv, r), a.vn[i]);
    }
    if (a.K8) {                                                // nn/mat.c:15-17: qrow_i8 per row
        float am = block_max_f32(fabsf(x), red32);
        float sc = quant_scale(am, 1e-12f), inv = __fdiv_rn(1.f, sc);
        if (i < hd) a.K8[slotp * hd + i] = (int8_t)quant_code(x, inv);
        if (i == 0) a.Ks[slotp] = sc;
        am = block_max_f32(fabsf(vv), red32);
        sc = quant_scale(am, 1e-12f); inv = __fdiv_rn(1.f, sc);
        if (i < hd) a.V8[slotp * hd + i] = (int8_t)quant_code(vv, inv);
        if (i == 0) a.Vs[slotp] = sc;
    } else if (i < hd) {
        a.K[slotp * hd + i] = x;
        a.V[slotp * hd + i] = vv;
    }
}

// Scores, softmax and accumulation.  A CTA takes one token, up to AT_G query heads that share a KV head (the key and
// value rows are read once for all of them) and one split of the positions 0..qpos; it walks its positions in
// sub-chunks of AT_CH with a running maximum and sum (the softmax of hw/hw_ops.h:22-26 evaluated piecewise:
// exp(s - m) terms are rescaled when the maximum moves), so shared memory does not grow with the context.  With one
// split the CTA writes ctx itself; otherwise it leaves {m, l, acc[hd]} per head in `part` and attn_merge_kernel joins
// the splits.  Decode steps (few tokens, long context) are split so that every SM has work; prompts are not.
constexpr int AT_CH = 128, AT_G = 4, AT_PB = 8, AT_WARPS = 8;

// four consecutive dimensions of a cached row as floats: f32 cache or int8 cache (codes only; the row scale is applied
// by the caller as the reference does, nn/attn_kernels.c:16,31)
__device__ __forceinline__ float4 attn_row4(const float *f, const int8_t *q, size_t off) {
    if (q) {
        const char4 c = *reinterpret_cast<const char4 *>(q + off);
        return make_float4((float)c.x, (float)c.y, (float)c.z, (float)c.w);
    }
    return *reinterpret_cast<const float4 *>(f + off);
}

// N per-lane partial sums (N = 16 or 32) -> lane L holds the total of value L >> (5 - log2 N)
template <int N>
__device__ __forceinline__ void attn_reduce(float (&v)[N], int lane) {
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) {
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            const bool up = (lane & off) != 0;
            const float send = up ? v[i] : v[i + n / 2];
            const float keep = up ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

// NV = float4 rounds a lane needs to cover a head: lane l holds dimensions 128 r + 4 l .. + 3 (head_dim <= 128 NV)
// NH = query heads whose dots are formed per key row (2 when a KV head serves at most two, else 4)
// FUSE (one token, position on the device): the work of attn_prep_kernel happens here, so a decode step is one launch
// less.  Every CTA norms and rotates its own query heads into shared memory (a warp per head; q and k in global memory
// are left as they came), and the CTA whose positions include the token's own also norms and rotates the key row and
// stores key and value rows in the cache before the block-wide barrier; it then reads them back like any other row.
template <int NV, int NH, bool FUSE>
__global__ void __launch_bounds__(AT_WARPS * 32, NV == 1 ? 3 : 1) attn_flash_kernel(AttnArgs a, int nsplit, int span, float *part) {
    extern __shared__ float sm_attn[];
    __shared__ float m_s[AT_G], l_s[AT_G], f_s[AT_G];
    const int hd = a.hd, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.H / a.KV, ngy = (G + AT_G - 1) / AT_G;
    const int s = blockIdx.z, kvh = blockIdx.y / ngy, g0 = (blockIdx.y - kvh * ngy) * AT_G, split = blockIdx.x;
    const int ng = G - g0 < AT_G ? G - g0 : AT_G, head0 = kvh * G + g0;
    int n = a.pos_base + s + 1;                                         // positions 0..qpos (re-read after the wait when it lives on the device)
    int t_lo = split * span;
    int t_hi = t_lo + span < n ? t_lo + span : n;
    const size_t base = (size_t)kvh * a.max_t;
    float *qs = sm_attn, *sc = qs + AT_G * NV * 128, *ps = sc + AT_G * AT_CH;   // q[AT_G][NV*128], sc[AT_G][AT_CH], partial[warps][AT_G][NV*128]
    // FUSE: warps past AT_G form the rotation table; theta^(2 j / rot) needs no input, so it is ready before the wait
    constexpr int ROPE_T = (AT_WARPS - AT_G - 1) * 32;                  // rot / 2 <= 128 <= 2 ROPE_T
    float den0 = 1.f, den1 = 1.f;
    if (FUSE && warp > AT_G) {
        const int jj = tid - (AT_G + 1) * 32;
        if (a.gemma) {                                                  // engines/gemma.c:290: theta^(-2j/hd), a factor
            den0 = powf(a.theta, __fdiv_rn(__fmul_rn(-2.0f, (float)jj), (float)hd));
            den1 = powf(a.theta, __fdiv_rn(__fmul_rn(-2.0f, (float)(jj + ROPE_T)), (float)hd));
        } else {                                                        // nn/rope.c:41: theta^(2j/rot), a divisor
            den0 = powf(a.theta, __fdiv_rn((float)(2 * jj), (float)a.rot));
            den1 = powf(a.theta, __fdiv_rn((float)(2 * (jj + ROPE_T)), (float)a.rot));
        }
    }
    pdl_trigger();
    pdl_wait();                                                         // rotated q and the cache rows of this call come from attn_prep_kernel (without FUSE)
    if (a.pos_dev) {
        int p0 = *a.pos_dev;                                            // clamped to [0, pos_base] like attn_prep_kernel does
        if (p0 < 0 || p0 > a.pos_base) { if (tid == 0 && a.err) atomicExch(a.err, 1); p0 = p0 < 0 ? 0 : a.pos_base; }
        n = p0 + s + 1; t_hi = t_lo + span < n ? t_lo + span : n;
    }
    if (a.window > 0 && n > a.window) {                                 // a sliding layer: positions qpos - window + 1 .. qpos (engines/gemma.c:373)
        t_lo += n - a.window;
        t_hi = t_lo + span < n ? t_lo + span : n;
    }
    if (FUSE) {
        const int pos = n - 1;
        const bool own = pos >= t_lo && pos < t_lo + span;
        for (int i = ng * NV * 128 + tid; i < AT_G * NV * 128; i += AT_WARPS * 32) qs[i] = 0.f;
        constexpr int NJ = NV * 4;                                      // lane l holds dimensions l + 32 j
        const bool mine = warp < ng || (warp == AT_G && own), isq = warp < ng;
        // pairs (j, j + half), nang of them rotated: nn/rope.c:39-49 (half = nang = rot / 2) or engines/gemma.c:287-297
        // (half = hd / 2, nang = rot)
        const int half = a.gemma ? hd / 2 : a.rot / 2, nang = a.gemma ? a.rot : a.rot / 2;
        float *xs = ps + warp * (NV * 128);
        float x[NJ];
        if (mine) {
            const float *row = isq ? a.q + (size_t)(head0 + warp) * hd : a.k + (size_t)kvh * hd;
            const float *nw = isq ? a.qn : a.kn;
            double ss = 0.0;
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int d = lane + 32 * j;
                x[j] = d < hd ? row[d] : 0.f;
                ss += (double)x[j] * (double)x[j];
            }
            if (nw) {                                                   // hw/hw_ops.h:14-18
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ss / hd), a.eps)));
#pragma unroll
                for (int j = 0; j < NJ; j++) {
                    const int d = lane + 32 * j;
                    if (d < hd) x[j] = __fmul_rn(__fmul_rn(x[j], r), nw[d]);
                }
            }
#pragma unroll
            for (int j = 0; j < NJ; j++) xs[lane + 32 * j] = x[j];
        } else if (warp > AT_G) {                                       // the other warps: cos and sin of the rot / 2 angles, once
            const int jj = tid - (AT_G + 1) * 32;                       // nn/rope.c:39-44
            if (jj < nang) { const float an = a.gemma ? __fmul_rn((float)pos, den0) : __fdiv_rn((float)pos, den0); sc[jj] = cosf(an); sc[128 + jj] = sinf(an); }
            if (jj + ROPE_T < nang) {
                const float an = a.gemma ? __fmul_rn((float)pos, den1) : __fdiv_rn((float)pos, den1);
                sc[jj + ROPE_T] = cosf(an); sc[128 + jj + ROPE_T] = sinf(an);
            }
        }
        __syncthreads();
        if (mine) {
#pragma unroll
            for (int j = 0; j < NJ; j++) {                              // nn/rope.c:45-49
                const int d = lane + 32 * j;
                const int jj = d < half ? d : d - half;
                if (d < 2 * half && jj < nang) {
                    const float c = sc[jj], sn = sc[128 + jj];
                    const float lo = xs[jj], hi = xs[jj + half];
                    x[j] = d < half ? __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn)) : __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
                }
            }
            if (isq) {
#pragma unroll
                for (int j = 0; j < NJ; j++) qs[warp * NV * 128 + lane + 32 * j] = x[j];   // zero past the head
            } else {                                                    // KV store (nn/attn.c:49-60)
                const size_t slotp = base + pos;
                float vv[NJ];
#pragma unroll
                for (int j = 0; j < NJ; j++) vv[j] = lane + 32 * j < hd ? a.v[(size_t)kvh * hd + lane + 32 * j] : 0.f;
                if (a.vn) {                                             // gemma's value norm (engines/gemma.c:320-324)
                    double sv2 = 0.0;
#pragma unroll
                    for (int j = 0; j < NJ; j++) sv2 += (double)vv[j] * (double)vv[j];
                    for (int off = 16; off > 0; off >>= 1) sv2 += __shfl_xor_sync(0xffffffffu, sv2, off);
                    const float rv = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(sv2 / hd), a.eps)));
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int d = lane + 32 * j;
                        if (d < hd) vv[j] = __fmul_rn(__fmul_rn(vv[j], rv), a.vn[d]);
                    }
                }
                if (a.K8) {                                             // nn/mat.c:15-17: qrow_i8 per row
                    float ak = 0.f, av = 0.f;
#pragma unroll
                    for (int j = 0; j < NJ; j++) { ak = fmaxf(ak, fabsf(x[j])); av = fmaxf(av, fabsf(vv[j])); }
                    for (int off = 16; off > 0; off >>= 1) {
                        ak = fmaxf(ak, __shfl_xor_sync(0xffffffffu, ak, off));
                        av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, off));
                    }
                    const float sk = quant_scale(ak, 1e-12f), ik = __fdiv_rn(1.f, sk);
                    const float sv = quant_scale(av, 1e-12f), iv = __fdiv_rn(1.f, sv);
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int d = lane + 32 * j;
                        if (d < hd) {
                            a.K8[slotp * hd + d] = (int8_t)quant_code(x[j], ik);
                            a.V8[slotp * hd + d] = (int8_t)quant_code(vv[j], iv);
                        }
                    }
                    if (lane == 0) { a.Ks[slotp] = sk; a.Vs[slotp] = sv; }
                } else {
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        const int d = lane + 32 * j;
                        if (d < hd) { a.K[slotp * hd + d] = x[j]; a.V[slotp * hd + d] = vv[j]; }
                    }
                }
            }
        }
    } else {
        for (int i = tid; i < AT_G * NV * 128; i += AT_WARPS * 32) {
            const int g = i / (NV * 128), dd = i - g * (NV * 128);
            qs[i] = g < ng && dd < hd ? a.q[(size_t)s * a.H * hd + (size_t)(head0 + g) * hd + dd] : 0.f;
        }
    }
    if (tid < AT_G) { m_s[tid] = -1e30f; l_s[tid] = 0.f; }
    bool dv[NV];                                                        // does round r of this lane lie inside the head
#pragma unroll
    for (int r = 0; r < NV; r++) dv[r] = r * 128 + lane * 4 < hd;
    float4 acc[AT_G][NV];
#pragma unroll
    for (int g = 0; g < AT_G; g++)
#pragma unroll
        for (int r = 0; r < NV; r++) acc[g][r] = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    for (int c0 = t_lo; c0 < t_hi; c0 += AT_CH) {
        const int nc = t_hi - c0 < AT_CH ? t_hi - c0 : AT_CH;
        // scores (hw/hw_ops.h:53-55; int8 keys nn/attn_kernels.c:14-17): a warp takes AT_PB positions at a time, all their
        // key rows requested before the first dot
        for (int tb = warp * AT_PB; tb < nc; tb += AT_WARPS * AT_PB) {
            float4 kr[AT_PB][NV];
#pragma unroll
            for (int u = 0; u < AT_PB; u++) {
                const size_t row = base + c0 + (tb + u < nc ? tb + u : nc - 1);
#pragma unroll
                for (int r = 0; r < NV; r++)
                    kr[u][r] = dv[r] ? attn_row4(a.K, a.K8, row * hd + r * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            // the lane's share of all AT_PB x NH dots, then ONE butterfly that leaves dot number L (NH = 4) or L / 2 in lane L
            // (31 shuffles for 32 dots instead of five per dot); value u * NH + g = position tb + u, head g
            float dsum[AT_PB * NH];
#pragma unroll
            for (int u = 0; u < AT_PB; u++)
#pragma unroll
                for (int g = 0; g < NH; g++) {
                    float d = 0.f;
#pragma unroll
                    for (int r = 0; r < NV; r++) {
                        const float4 q4 = *reinterpret_cast<const float4 *>(qs + g * NV * 128 + r * 128 + lane * 4);   // zero rows for g >= ng
                        d = fmaf(q4.x, kr[u][r].x, d); d = fmaf(q4.y, kr[u][r].y, d);
                        d = fmaf(q4.z, kr[u][r].z, d); d = fmaf(q4.w, kr[u][r].w, d);
                    }
                    dsum[u * NH + g] = d;
                }
            attn_reduce<AT_PB * NH>(dsum, lane);
            {
                const int val = NH == 4 ? lane : lane >> 1, u = val / NH, g = val - u * NH;
                if (tb + u < nc && g < ng && (NH == 4 || !(lane & 1))) {
                    const float d = dsum[0];
                    sc[g * AT_CH + tb + u] = a.K8 ? __fmul_rn(__fmul_rn(a.Ks[base + c0 + tb + u], d), a.scale) : __fmul_rn(d, a.scale);
                }
            }
        }
        __syncthreads();
        // running maximum and sum: warp g looks after head g
        if (warp < ng) {
            float mc = -1e30f;
            for (int t = lane; t < nc; t += 32) mc = fmaxf(mc, sc[warp * AT_CH + t]);
            for (int off = 16; off > 0; off >>= 1) mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, off));
            const float m_old = m_s[warp], m_new = fmaxf(m_old, mc);
            float sum = 0.f;
            for (int t = lane; t < nc; t += 32) {
                const float e = expf(__fsub_rn(sc[warp * AT_CH + t], m_new));
                sc[warp * AT_CH + t] = e; sum += e;
            }
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (lane == 0) {
                const float f = expf(__fsub_rn(m_old, m_new));              // 0 on the first sub-chunk, 1 when the maximum stays
                f_s[warp] = f; m_s[warp] = m_new; l_s[warp] = fmaf(l_s[warp], f, sum);
            }
        }
        __syncthreads();
        // accumulation (hw/hw_ops.h:56-59; int8 values nn/attn_kernels.c:26-35): the warps take the positions in turn,
        // AT_PB value rows requested at a time
#pragma unroll
        for (int g = 0; g < AT_G; g++) {
            const float f = g < ng ? f_s[g] : 0.f;
#pragma unroll
            for (int r = 0; r < NV; r++) { acc[g][r].x *= f; acc[g][r].y *= f; acc[g][r].z *= f; acc[g][r].w *= f; }
        }
        for (int tb = warp * AT_PB; tb < nc; tb += AT_WARPS * AT_PB) {
            float4 vr[AT_PB][NV];
#pragma unroll
            for (int u = 0; u < AT_PB; u++) {
                const size_t row = base + c0 + (tb + u < nc ? tb + u : nc - 1);
#pragma unroll
                for (int r = 0; r < NV; r++)
                    vr[u][r] = dv[r] ? attn_row4(a.V, a.V8, row * hd + r * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < AT_PB; u++) {
                if (tb + u >= nc) break;
                const float vs = a.V8 ? a.Vs[base + c0 + tb + u] : 1.f;
#pragma unroll
                for (int g = 0; g < AT_G; g++) {
                    if (g >= ng) break;
                    const float p = sc[g * AT_CH + tb + u];
                    const float w = a.V8 ? __fmul_rn(p, vs) : p;            // nn/attn_kernels.c:31: a = sc * Vs
#pragma unroll
                    for (int r = 0; r < NV; r++) {
                        acc[g][r].x = fmaf(w, vr[u][r].x, acc[g][r].x); acc[g][r].y = fmaf(w, vr[u][r].y, acc[g][r].y);
                        acc[g][r].z = fmaf(w, vr[u][r].z, acc[g][r].z); acc[g][r].w = fmaf(w, vr[u][r].w, acc[g][r].w);
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int g = 0; g < AT_G; g++)
#pragma unroll
        for (int r = 0; r < NV; r++)
            *reinterpret_cast<float4 *>(ps + ((size_t)warp * AT_G + g) * NV * 128 + r * 128 + lane * 4) = acc[g][r];
    __syncthreads();
    for (int i = tid; i < ng * hd; i += AT_WARPS * 32) {
        const int g = i / hd, dd = i - g * hd;
        float tot = ps[(size_t)g * NV * 128 + dd];
        for (int w = 1; w < AT_WARPS; w++) tot += ps[((size_t)w * AT_G + g) * NV * 128 + dd];
        if (nsplit == 1) {
            a.ctx[(size_t)s * a.H * hd + (size_t)(head0 + g) * hd + dd] = __fdiv_rn(tot, l_s[g]);
        } else {
            float *p = part + (((size_t)s * a.H + head0 + g) * nsplit + split) * (hd + 2);
            p[2 + dd] = tot;
            if (dd == 0) { p[0] = m_s[g]; p[1] = l_s[g]; }
        }
    }
}

// Prompts.  A CTA takes 32 query rows that share every key and value row: consecutive tokens x the
// query heads of one KV head (8 tokens x 4 heads, 16 x 2 or 32 x 1).  The positions are walked 64 at a time: the sub-chunk's key and value rows
// are staged in shared memory once (int8 rows as their codes, scales aside), the 32 x 64 scores are register-tiled
// dot products from shared memory (thread = one position x eight rows, no shuffles), one warp per token keeps the
// running maximum and sum of its four rows, and the same warp accumulates its token's rows over the staged value
// rows (lane = four dimensions per 128).  Causal: a position past a token's own scores -1e30 and weighs 0; a sliding
// layer starts at the first sub-chunk any of the CTA's tokens can see.  HD = 128 (two CTAs per SM) or 256 (one).
constexpr int AP_CH = 64, AP_PP = AP_CH + 4;
template <int HD> struct ApL {
    static constexpr int KP = HD + 4;
    static constexpr size_t SMEM = ((size_t)32 * KP + (size_t)AP_CH * KP + (size_t)AP_CH * HD + (size_t)32 * AP_PP + 2 * AP_CH + 3 * 32) * 4;
};

template <int HD>
__global__ void __launch_bounds__(256, HD == 128 ? 2 : 1) attn_prompt_kernel(AttnArgs a) {
    constexpr int AP_KP = ApL<HD>::KP, NQ4 = HD / 4, NV = HD / 128;
    extern __shared__ float sm_attn[];
    float *Qs = sm_attn;                                  // [32][AP_KP]   row = token * 4 + head
    float *Kc = Qs + 32 * AP_KP;                          // [AP_CH][AP_KP]
    float *Vc = Kc + AP_CH * AP_KP;                       // [AP_CH][HD]
    float *P = Vc + AP_CH * HD;                           // [32][AP_PP]   scores, then weights
    float *ksc = P + 32 * AP_PP, *vsc = ksc + AP_CH;      // row scales of an int8 cache
    float *m_s = vsc + AP_CH, *l_s = m_s + 32, *f_s = l_s + 32;
    (void)f_s;
    const int hd = a.hd, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = a.H / a.KV, ngy = (G + AT_G - 1) / AT_G;
    const int kvh = blockIdx.y / ngy, g0 = (blockIdx.y - kvh * ngy) * AT_G;
    const int ng = G - g0 < AT_G ? G - g0 : AT_G, head0 = kvh * G + g0;
    // the 32 query rows are (32 / ngp) tokens x ngp heads, ngp = the head count rounded up to 1, 2 or 4: row = token * ngp + head
    const int ngc = G < AT_G ? G : AT_G;                  // (the same for every CTA of the launch; a last group may have fewer heads)
    const int lg = ngc > 2 ? 2 : ngc - 1, ngp = 1 << lg, tq = 32 >> lg;
    const int s0 = blockIdx.x * tq;
    const int ntok = a.S - s0 < tq ? a.S - s0 : tq;
    const int n_all = a.pos_base + s0 + ntok;             // positions 0 .. the last token's own
    const size_t base = (size_t)kvh * a.max_t;
    pdl_trigger();
    pdl_wait();
    for (int i = tid; i < 32 * HD; i += 256) {
        const int row = i / HD, dd = i - row * HD, tok = row >> lg, g = row & (ngp - 1);
        Qs[row * AP_KP + dd] = tok < ntok && g < ng && dd < hd ? a.q[(size_t)(s0 + tok) * a.H * hd + (size_t)(head0 + g) * hd + dd] : 0.f;
    }
    if (tid < 32) { m_s[tid] = -1e30f; l_s[tid] = 0.f; }
    float4 acc[4][NV];                                    // this warp's token, heads 0..3, dimensions 128 r + 4 lane .. + 3
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int r = 0; r < NV; r++) acc[j][r] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int p_me = tid & 63, rg = tid >> 6;             // scores: my position in the sub-chunk, my eight rows rg * 8 ..
    const int hd4 = hd >> 2;
    // a sliding layer: the CTA's first token sees positions from (pos_base + s0) - window + 1 on, the later ones from further on
    int c_first = 0;
    if (a.window > 0 && a.pos_base + s0 - a.window + 1 > 0) c_first = (a.pos_base + s0 - a.window + 1) / AP_CH * AP_CH;
    for (int c0 = c_first; c0 < n_all; c0 += AP_CH) {
        const int nc = n_all - c0 < AP_CH ? n_all - c0 : AP_CH;
        __syncthreads();                                  // everyone is done with the previous sub-chunk (and Qs is written)
        for (int i = tid; i < AP_CH * NQ4; i += 256) {    // stage: position i / NQ4, dimensions 4 (i % NQ4) ..
            const int pp = i / NQ4, q4 = i - pp * NQ4;
            float4 kv = make_float4(0.f, 0.f, 0.f, 0.f), vv = kv;
            if (pp < nc && q4 < hd4) {
                const size_t off = (base + c0 + pp) * hd + q4 * 4;
                kv = attn_row4(a.K, a.K8, off); vv = attn_row4(a.V, a.V8, off);
            }
            *reinterpret_cast<float4 *>(Kc + pp * AP_KP + q4 * 4) = kv;
            *reinterpret_cast<float4 *>(Vc + pp * HD + q4 * 4) = vv;
        }
        if (tid < AP_CH) {
            ksc[tid] = a.K8 && tid < nc ? a.Ks[base + c0 + tid] : 1.f;
            vsc[tid] = a.V8 && tid < nc ? a.Vs[base + c0 + tid] : 1.f;
        }
        __syncthreads();
        {   // scores (hw/hw_ops.h:53-55; int8 keys nn/attn_kernels.c:14-17)
            float d8[8];
#pragma unroll
            for (int j = 0; j < 8; j++) d8[j] = 0.f;
            const float *kp = Kc + p_me * AP_KP, *qp = Qs + rg * 8 * AP_KP;
            for (int k4 = 0; k4 < hd4; k4++) {
                const float4 kv = *reinterpret_cast<const float4 *>(kp + k4 * 4);
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float4 qv = *reinterpret_cast<const float4 *>(qp + j * AP_KP + k4 * 4);
                    d8[j] = fmaf(qv.x, kv.x, d8[j]); d8[j] = fmaf(qv.y, kv.y, d8[j]);
                    d8[j] = fmaf(qv.z, kv.z, d8[j]); d8[j] = fmaf(qv.w, kv.w, d8[j]);
                }
            }
            const float ks = ksc[p_me];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int row = rg * 8 + j, tok = row >> lg;
                const int qpos = a.pos_base + s0 + tok;
                const bool seen = p_me < nc && c0 + p_me <= qpos && (a.window <= 0 || c0 + p_me > qpos - a.window);
                const float v = a.K8 ? __fmul_rn(__fmul_rn(ks, d8[j]), a.scale) : __fmul_rn(d8[j], a.scale);
                P[row * AP_PP + p_me] = seen ? v : -1e30f;
            }
        }
        __syncthreads();
        // warp = token: running maximum and sum of its four rows (hw/hw_ops.h:22-26, piecewise), weights in place
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float *row = P + (warp * 4 + j) * AP_PP;
            const float x0 = row[lane], x1 = row[lane + 32];
            float mc = fmaxf(x0, x1);
            for (int off = 16; off > 0; off >>= 1) mc = fmaxf(mc, __shfl_xor_sync(0xffffffffu, mc, off));
            const float m_old = m_s[warp * 4 + j], m_new = fmaxf(m_old, mc);
            const float e0 = x0 <= -1e30f ? 0.f : expf(__fsub_rn(x0, m_new)), e1 = x1 <= -1e30f ? 0.f : expf(__fsub_rn(x1, m_new));
            float sum = e0 + e1;
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            const float f = expf(__fsub_rn(m_old, m_new));
            // int8 values: a = weight * Vs (nn/attn_kernels.c:31)
            row[lane] = a.V8 ? __fmul_rn(e0, vsc[lane]) : e0;
            row[lane + 32] = a.V8 ? __fmul_rn(e1, vsc[lane + 32]) : e1;
            __syncwarp();
            if (lane == 0) { m_s[warp * 4 + j] = m_new; l_s[warp * 4 + j] = fmaf(l_s[warp * 4 + j], f, sum); }
#pragma unroll
            for (int r = 0; r < NV; r++) { acc[j][r].x *= f; acc[j][r].y *= f; acc[j][r].z *= f; acc[j][r].w *= f; }
        }
        __syncwarp();
        // accumulation (hw/hw_ops.h:56-59): this warp's token over the staged value rows, lane = four dimensions per 128
        {
            const float *pr = P + warp * 4 * AP_PP;
            for (int pp = 0; pp < nc; pp++) {
                float w4[4];
#pragma unroll
                for (int j = 0; j < 4; j++) w4[j] = pr[j * AP_PP + pp];
#pragma unroll
                for (int r = 0; r < NV; r++) {
                    if (r * 32 + lane < hd4) {
                        const float4 vv = *reinterpret_cast<const float4 *>(Vc + pp * HD + (r * 32 + lane) * 4);
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            acc[j][r].x = fmaf(w4[j], vv.x, acc[j][r].x); acc[j][r].y = fmaf(w4[j], vv.y, acc[j][r].y);
                            acc[j][r].z = fmaf(w4[j], vv.z, acc[j][r].z); acc[j][r].w = fmaf(w4[j], vv.w, acc[j][r].w);
                        }
                    }
                }
            }
        }
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < NV; r++) {
        if (r * 32 + lane >= hd4) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int row = warp * 4 + j, tok = row >> lg, g = row & (ngp - 1);
            if (tok >= ntok || g >= ng) continue;
            const float l = l_s[row];
            float4 o = acc[j][r];
            o.x = __fdiv_rn(o.x, l); o.y = __fdiv_rn(o.y, l); o.z = __fdiv_rn(o.z, l); o.w = __fdiv_rn(o.w, l);
            *reinterpret_cast<float4 *>(a.ctx + (size_t)(s0 + tok) * a.H * hd + (size_t)(head0 + g) * hd + (r * 32 + lane) * 4) = o;
        }
    }
}

// joins the splits of one (token, head): M = max m_c, ctx = sum acc_c exp(m_c - M) / sum l_c exp(m_c - M)
__global__ void __launch_bounds__(256) attn_merge_kernel(AttnArgs a, int nsplit, const float *part) {
    extern __shared__ float fm[];                                       // per split: its factor exp(m_c - M), 0 for an empty one
    __shared__ float red32[8];
    const int s = blockIdx.x, hh = blockIdx.y, hd = a.hd, tid = threadIdx.x, nth = blockDim.x;
    const float *p = part + ((size_t)s * a.H + hh) * nsplit * (hd + 2);
    pdl_trigger();
    pdl_wait();
    float m = -1e30f;
    for (int c = tid; c < nsplit; c += nth) { fm[c] = p[(size_t)c * (hd + 2)]; m = fmaxf(m, fm[c]); }
    const float M = block_max_f32(m, red32);
    float l = 0.f;
    for (int c = tid; c < nsplit; c += nth) {
        const float lc = p[(size_t)c * (hd + 2) + 1];
        const float f = lc == 0.f ? 0.f : expf(__fsub_rn(fm[c], M));     // a split past the token's position has nothing in it
        fm[c] = f; l = fmaf(lc, f, l);
    }
    const float L = block_sum_f32(l, red32);                             // (its barriers also publish fm)
    if (tid < hd) {
        float acc = 0.f;
        for (int c0 = 0; c0 < nsplit; c0 += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = c0 + u < nsplit ? p[(size_t)(c0 + u) * (hd + 2) + 2 + tid] : 0.f;
#pragma unroll
            for (int u = 0; u < 8; u++) if (c0 + u < nsplit) acc = fmaf(v[u], fm[c0 + u], acc);
        }
        a.ctx[(size_t)s * a.H * hd + (size_t)hh * hd + tid] = __fdiv_rn(acc, L);
    }
}

// the gated variant's last step (nn/attn.c:68-69): ctx[i] *= 1 / (1 + expf(-gate[i]))
__global__ void __launch_bounds__(256) attn_gate_kernel(float *ctx, const float *gate, long long n) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) ctx[i] = __fmul_rn(ctx[i], __fdiv_rn(1.f, __fadd_rn(1.f, moty_expf(-gate[i]))));
}

}  // namespace

int launch_attn_gate(float *ctx, const float *gate, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    CK(moty_launch_pdl(attn_gate_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, st, ctx, gate, n));
    return 0;
}

// room for the partial results of a call whose positions are split (at most 3 * sms + 1 splits in all)
size_t attn_scratch_bytes(int S, int H, int KV, int hd, int sms) {
    const int G = H / KV, ngy = (G + AT_G - 1) / AT_G;
    const long long units = (long long)S * KV * ngy;
    if (units >= 2LL * sms) return 0;
    const long long nsplit = (3LL * sms + units - 1) / units + 1;
    return (size_t)S * H * nsplit * (hd + 2) * 4;
}

// q, k: modified in place (normed, rotated), as the reference does.  Caches: f32 (K, V) or int8 (K8, V8, Ks, Vs).
// part: scratch of attn_scratch_bytes(...) for decode-sized calls (null: never split the positions).
// pos_dev: null, or a device int holding the first position; pos_base is then the LARGEST value it may take (it sizes
// the launch, so that one captured launch serves every position up to it).
int launch_attn_core(float *ctx, float *q, float *k, const float *v, int S, int pos_base, int H, int KV, int hd, int rot,
                     float theta, float eps, const float *qn, const float *kn, float *K, float *V, int8_t *K8, int8_t *V8,
                     float *Ks, float *Vs, int max_t, float *part, const int *pos_dev, int *err, int sms, cudaStream_t st,
                     int gemma, int window, float scale, const float *vn) {
    if (S <= 0) return 0;
    const bool rot_bad = gemma ? (rot < 0 || rot > hd / 2) : (rot < 0 || rot > hd || (rot & 1));
    if (hd <= 0 || hd > 256 || hd % 4 || rot_bad || H <= 0 || KV <= 0 || H % KV || pos_base < 0 || window < 0 ||
        pos_base + S > max_t)
        return moty_set_error(MOTY_CUDA_EARG, "attn_core: S=%d pos=%d max_t=%d H=%d KV=%d hd=%d rot=%d", S, pos_base, max_t, H, KV, hd, rot);
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.ctx = ctx; a.qn = qn; a.kn = kn; a.K = K; a.V = V; a.K8 = K8; a.V8 = V8; a.Ks = Ks; a.Vs = Vs;
    a.S = S; a.pos_base = pos_base; a.H = H; a.KV = KV; a.hd = hd; a.rot = rot; a.max_t = max_t;
    a.theta = theta; a.eps = eps; a.scale = scale > 0.f ? scale : 1.f / sqrtf((float)hd); a.pos_dev = pos_dev; a.err = err;
    a.gemma = gemma; a.window = window; a.vn = vn;
    const int nth_prep = (hd + 31) / 32 * 32;
    // one token at a position read from the device (a replayed decode step): norm, rotation and cache store ride in the
    // scores launch, and q and k are not written back
    const bool fuse = pos_dev && S == 1;
    if (!fuse) CK(moty_launch_pdl(attn_prep_kernel, dim3(S, H + KV), dim3(nth_prep), (size_t)0, st, a));
    const int NVr = hd > 128 ? 2 : 1;
    const size_t smem = ((size_t)AT_G * NVr * 128 + (size_t)AT_G * AT_CH + (size_t)AT_WARPS * AT_G * NVr * 128) * 4;
    const int G = H / KV, ngy = (G + AT_G - 1) / AT_G;
    const int T = window > 0 && pos_base + S > window ? window : pos_base + S;      // the most positions any token attends to
    // prompts: eight tokens per CTA share staged key and value rows, when that still gives every SM a CTA
    const int ng_cta = G < AT_G ? G : AT_G, tq = ng_cta > 2 ? 8 : (ng_cta == 2 ? 16 : 32);
    const long long tiles = (long long)((S + tq - 1) / tq) * KV * ngy;
    if (S >= 8 && tiles >= sms && !pos_dev) {
        static bool attr_p[MOTY_MAX_DEV];
        int devp = 0;
        CK(cudaGetDevice(&devp));
        if (devp < 0 || devp >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "attn_core: device %d", devp);
        if (!attr_p[devp]) {
            CK(cudaFuncSetAttribute(attn_prompt_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ApL<128>::SMEM));
            CK(cudaFuncSetAttribute(attn_prompt_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ApL<256>::SMEM));
            attr_p[devp] = true;
        }
        const dim3 pgrid((S + tq - 1) / tq, KV * ngy);
        if (hd <= 128) CK(moty_launch_pdl(attn_prompt_kernel<128>, pgrid, dim3(256), ApL<128>::SMEM, st, a));
        else CK(moty_launch_pdl(attn_prompt_kernel<256>, pgrid, dim3(256), ApL<256>::SMEM, st, a));
        return 0;
    }
    // few (token, KV head) pairs: split the positions so that every SM gets a few CTAs
    int nsplit = 1;
    const long long units = (long long)S * KV * ngy;
    // A split's positions come in multiples of one pass of the eight warps (64; with 128, the sub-chunk, a context of
    // 500-1000 positions got too few CTAs: 32 query / 4 KV heads at 513 12.3 -> 9.9 us, 16 / 8 at 1000 11.2 -> 10.1 us;
    // 32 measured worse).  Three resident sets of CTAs for heads of up to 128, two for wider ones (one CTA per SM there:
    // 8192 positions 52 -> 44 us, 32768 129 -> 119 us; a single set is better around 2000-4000 and much worse beyond).
    constexpr int gran = AT_PB * AT_WARPS;
    if (units < 2LL * sms && T > 2 * AT_CH) {                           // (a context of two sub-chunks is not worth a merge launch)
        nsplit = (int)(((NVr == 1 ? 3LL : 2LL) * sms + units - 1) / units);
        const int most = (T + gran - 1) / gran;
        if (nsplit > most) nsplit = most;
        if (nsplit < 1) nsplit = 1;
    }
    int span = (T + nsplit - 1) / nsplit;
    span = (span + gran - 1) / gran * gran;
    nsplit = (T + span - 1) / span;
    if (nsplit > 1 && !part) return moty_set_error(MOTY_CUDA_EARG, "attn_core: scratch for %d splits missing", nsplit);
    static bool attr_done[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "attn_core: device %d", dev);
    if (!attr_done[dev]) {
        CK(cudaFuncSetAttribute(attn_flash_kernel<1, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<1, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<2, 2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<2, 4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<1, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<1, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<2, 2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        CK(cudaFuncSetAttribute(attn_flash_kernel<2, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
        attr_done[dev] = true;
    }
    if ((unsigned)S > 65535u) return moty_set_error(MOTY_CUDA_ELIMIT, "attn_core: S=%d in one call", S);
    const dim3 fgrid(nsplit, KV * ngy, S), fblock(AT_WARPS * 32);
    if (fuse) {
        if (NVr == 1 && G <= 2) CK(moty_launch_pdl(attn_flash_kernel<1, 2, true>, fgrid, fblock, smem, st, a, nsplit, span, part));
        else if (NVr == 1) CK(moty_launch_pdl(attn_flash_kernel<1, 4, true>, fgrid, fblock, smem, st, a, nsplit, span, part));
        else if (G <= 2) CK(moty_launch_pdl(attn_flash_kernel<2, 2, true>, fgrid, fblock, smem, st, a, nsplit, span, part));
        else CK(moty_launch_pdl(attn_flash_kernel<2, 4, true>, fgrid, fblock, smem, st, a, nsplit, span, part));
    } else if (NVr == 1 && G <= 2) CK(moty_launch_pdl(attn_flash_kernel<1, 2, false>, fgrid, fblock, smem, st, a, nsplit, span, part));
    else if (NVr == 1) CK(moty_launch_pdl(attn_flash_kernel<1, 4, false>, fgrid, fblock, smem, st, a, nsplit, span, part));
    else if (G <= 2) CK(moty_launch_pdl(attn_flash_kernel<2, 2, false>, fgrid, fblock, smem, st, a, nsplit, span, part));
    else CK(moty_launch_pdl(attn_flash_kernel<2, 4, false>, fgrid, fblock, smem, st, a, nsplit, span, part));
    if (nsplit > 1)
        CK(moty_launch_pdl(attn_merge_kernel, dim3(S, H), dim3(nth_prep), (size_t)nsplit * 4, st, a, nsplit, (const float *)part));
    return 0;
}
