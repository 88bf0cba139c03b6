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
    const bool isq = slot < a.H;
    const int hh = isq ? slot : slot - a.H;
    float *row = isq ? a.q + (size_t)s * a.H * hd + (size_t)hh * hd : a.k + (size_t)s * a.KV * hd + (size_t)hh * hd;
    const float *nw = isq ? a.qn : a.kn;
    const int pos = a.pos_base + s;
    float x = i < hd ? row[i] : 0.f;
    if (nw) {                                                  // hw/hw_ops.h:14-18
        const double ms = block_sum_f64((double)x * (double)x, red64);
        const float r = __fdiv_rn(1.f, __fsqrt_rn(__fadd_rn((float)(ms / hd), a.eps)));
        if (i < hd) x = __fmul_rn(__fmul_rn(x, r), nw[i]);
    }
    if (i < hd) xs[i] = x;
    __syncthreads();
    const int half = a.rot / 2;
    if (i < a.rot) {                                           // nn/rope.c:39-49
        const int j = i < half ? i : i - half;
        const float angle = __fdiv_rn((float)pos, powf(a.theta, __fdiv_rn((float)(2 * j), (float)a.rot)));
        const float c = cosf(angle), sn = sinf(angle);
        const float lo = xs[j], hi = xs[j + half];
        x = i < half ? __fsub_rn(__fmul_rn(lo, c), __fmul_rn(hi, sn)) : __fadd_rn(__fmul_rn(lo, sn), __fmul_rn(hi, c));
    }
    if (i < hd) row[i] = x;
    if (isq) return;
    // KV store (nn/attn.c:49-60)
    const size_t slotp = (size_t)hh * a.max_t + pos;
    const float vv = i < hd ? a.v[(size_t)s * a.KV * hd + (size_t)hh * hd + i] : 0.f;
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

// One CTA per (token, query head): scores against positions 0..qpos, softmax, accumulation.
// Shared memory: q[hd], sc[n], partial[ngrp][hd].
__global__ void __launch_bounds__(256) attn_core_kernel(AttnArgs a) {
    extern __shared__ float sm_attn[];
    __shared__ float red32[8];
    const int s = blockIdx.x, hh = blockIdx.y, hd = a.hd, tid = threadIdx.x, nth = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarp = nth >> 5;
    const int kvh = hh / (a.H / a.KV), qpos = a.pos_base + s, n = qpos + 1;
    const size_t base = (size_t)kvh * a.max_t;
    float *qs = sm_attn, *sc = sm_attn + hd, *part = sc + (a.pos_base + a.S);
    const float *qv = a.q + (size_t)s * a.H * hd + (size_t)hh * hd;
    for (int i = tid; i < hd; i += nth) qs[i] = qv[i];
    __syncthreads();
    // scores (hw/hw_ops.h:53-55; int8 keys nn/attn_kernels.c:14-17): a warp per position
    for (int t = warp; t < n; t += nwarp) {
        float d = 0.f;
        if (a.K8) {
            const int8_t *kr = a.K8 + (base + t) * hd;
            for (int i = lane; i < hd; i += 32) d = fmaf(qs[i], (float)kr[i], d);
        } else {
            const float *kr = a.K + (base + t) * hd;
            for (int i = lane; i < hd; i += 32) d = fmaf(qs[i], kr[i], d);
        }
        for (int off = 16; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        if (lane == 0) sc[t] = a.K8 ? __fmul_rn(__fmul_rn(a.Ks[base + t], d), a.scale) : __fmul_rn(d, a.scale);
    }
    __syncthreads();
    // softmax (hw/hw_ops.h:22-26)
    float m = -1e30f;
    for (int t = tid; t < n; t += nth) m = fmaxf(m, sc[t]);
    m = block_max_f32(m, red32);
    float sum = 0.f;
    for (int t = tid; t < n; t += nth) { const float e = expf(__fsub_rn(sc[t], m)); sc[t] = e; sum += e; }
    sum = block_sum_f32(sum, red32);
    for (int t = tid; t < n; t += nth) sc[t] = __fdiv_rn(sc[t], sum);
    __syncthreads();
    // accumulation (hw/hw_ops.h:56-59; int8 values nn/attn_kernels.c:26-35): thread = dimension, groups of threads
    // take positions round-robin, partial sums are added in group order
    const int ngrp = nth / hd > 0 ? nth / hd : 1;
    const int grp = tid / hd, d = tid - grp * hd;
    if (grp < ngrp && d < hd) {
        float acc = 0.f;
        if (a.V8) {
            for (int t = grp; t < n; t += ngrp)
                acc = fmaf(__fmul_rn(sc[t], a.Vs[base + t]), (float)a.V8[(base + t) * hd + d], acc);
        } else {
            for (int t = grp; t < n; t += ngrp) acc = fmaf(sc[t], a.V[(base + t) * hd + d], acc);
        }
        part[grp * hd + d] = acc;
    }
    __syncthreads();
    if (tid < hd) {
        float acc = part[tid];
        for (int g = 1; g < ngrp; g++) acc += part[g * hd + tid];
        a.ctx[(size_t)s * a.H * hd + (size_t)hh * hd + tid] = acc;
    }
}

}  // namespace

// q, k: modified in place (normed, rotated), as the reference does.  Caches: f32 (K, V) or int8 (K8, V8, Ks, Vs).
int launch_attn_core(float *ctx, float *q, float *k, const float *v, int S, int pos_base, int H, int KV, int hd, int rot,
                     float theta, float eps, const float *qn, const float *kn, float *K, float *V, int8_t *K8, int8_t *V8,
                     float *Ks, float *Vs, int max_t, cudaStream_t st) {
    if (S <= 0) return 0;
    if (hd <= 0 || hd > 256 || rot < 0 || rot > hd || (rot & 1) || H <= 0 || KV <= 0 || H % KV || pos_base < 0 ||
        pos_base + S > max_t)
        return moty_set_error(MOTY_CUDA_EARG, "attn_core: S=%d pos=%d max_t=%d H=%d KV=%d hd=%d rot=%d", S, pos_base, max_t, H, KV, hd, rot);
    AttnArgs a;
    a.q = q; a.k = k; a.v = v; a.ctx = ctx; a.qn = qn; a.kn = kn; a.K = K; a.V = V; a.K8 = K8; a.V8 = V8; a.Ks = Ks; a.Vs = Vs;
    a.S = S; a.pos_base = pos_base; a.H = H; a.KV = KV; a.hd = hd; a.rot = rot; a.max_t = max_t;
    a.theta = theta; a.eps = eps; a.scale = 1.f / sqrtf((float)hd);
    const int nth_prep = (hd + 31) / 32 * 32;
    attn_prep_kernel<<<dim3(S, H + KV), nth_prep, 0, st>>>(a);
    CK(cudaGetLastError());
    const int nth = nth_prep > 128 ? nth_prep : 128;
    const int ngrp = nth / hd > 0 ? nth / hd : 1;
    const size_t smem = ((size_t)hd + (size_t)(pos_base + S) + (size_t)ngrp * hd) * 4;
    if (smem > 200 * 1024) return moty_set_error(MOTY_CUDA_ELIMIT, "attn_core: %d positions need %zu bytes of shared memory", pos_base + S, smem);
    static size_t attr_smem[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "attn_core: device %d", dev);
    if (smem > 48 * 1024 && smem > attr_smem[dev]) {
        CK(cudaFuncSetAttribute(attn_core_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_smem[dev] = 200 * 1024;
    }
    attn_core_kernel<<<dim3(S, H), nth, smem, st>>>(a);
    CK(cudaGetLastError());
    return 0;
}
