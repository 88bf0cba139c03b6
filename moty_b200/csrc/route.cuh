// route.cuh -- the MoE router of one token row, run by one warp.  Shared by the stand-alone
// router kernel (router.cu) and the fused decode kernels, so that both produce the same bits.
#pragma once
#include "common.cuh"

// order-preserving map float -> unsigned (larger float <=> larger key); -0 is folded into +0 first
// so that equal floats have equal keys
__device__ __forceinline__ unsigned route_key(float v) {
    unsigned u = __float_as_uint(v + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Softmax follows moty_hw_softmax_ref (hw/hw_ops.h:22-26): running maximum from -1e30,
// e = exp(x - m) rounded to f32, the sum taken SEQUENTIALLY in index order in f32 (every lane runs
// the same chain), then one true division per element.  exp is moty_expf (common.cuh), the
// restatement of the C library's expf, so the probabilities carry the reference's bits.
//
// Top-K follows moty_moe_topk (runtime/moecache.c:97-111): K rounds of "largest value not yet
// taken", strict > against a floor of -1e30, so equal values go to the lowest index.  The argmax
// with lowest-index tie-break is order independent: every lane scans its own slice in ascending
// order, the warp takes the largest key (one redux) and the lowest index that holds it (a second
// redux).  A taken entry is overwritten with -inf in the scratch row, which strict > never picks.
//
// lg: the E logits (global); p: E floats of scratch (shared memory, 16-byte aligned, clobbered);
// idx_out/w_out: K entries each (any address space); probs_out: E entries or null.

// the sequential softmax denominator: every lane runs the same chain of E additions over the
// scratch row; operands come in batches of 128-bit loads so that only the additions are serial
__device__ __forceinline__ float route_seq_sum(const float *p, int E) {
    float total = 0.f;
    const float4 *p4 = reinterpret_cast<const float4 *>(p);
    const int E4 = E >> 2;
    int e4 = 0;
    for (; e4 + 8 <= E4; e4 += 8) {
        float4 v[8];
#pragma unroll
        for (int q = 0; q < 8; q++) v[q] = p4[e4 + q];
#pragma unroll
        for (int q = 0; q < 8; q++) {
            total = __fadd_rn(total, v[q].x); total = __fadd_rn(total, v[q].y);
            total = __fadd_rn(total, v[q].z); total = __fadd_rn(total, v[q].w);
        }
    }
    for (int e = e4 * 4; e < E; e++) total = __fadd_rn(total, p[e]);
    return total;
}

// one round's winner over the lanes' local bests (bv, bi): largest value, lowest index among equals
__device__ __forceinline__ int route_pick(float bv, int bi, float &gv) {
    const unsigned key = bi >= 0 ? route_key(bv) : 0u;             // key 0 is below every real key (-inf maps to 0x007fffff)
    const unsigned kmax = __reduce_max_sync(0xffffffffu, key);
    const unsigned cand = (bi >= 0 && key == kmax) ? (unsigned)bi : 0xffffffffu;
    const unsigned win = __reduce_min_sync(0xffffffffu, cand);
    const int gi = win == 0xffffffffu ? -1 : (int)win;
    // the winning value, bit for bit, from the lane that owns it (lane = index mod 32)
    gv = __shfl_sync(0xffffffffu, bv, gi >= 0 ? (gi & 31) : 0);
    if (gi < 0) gv = -1e30f;
    return gi;
}

// E <= 32 * EPL: the row lives in registers (entry e = lane + 32 j in v[j]); everything is unrolled,
// so the f64 exponentials and the divisions of a lane overlap and the K rounds touch no memory.
template <int EPL>
__device__ __forceinline__ void route_row_warp_reg(const float *__restrict__ lg, int E, int K, float *p, int do_softmax,
                                                   int norm_topk, int lane, int *idx_out, float *w_out,
                                                   float *probs_out) {
    const float NEG_INF = __int_as_float(0xff800000);
    float v[EPL];
#pragma unroll
    for (int j = 0; j < EPL; j++) v[j] = lane + 32 * j < E ? lg[lane + 32 * j] : NEG_INF;
    if (do_softmax) {
        float m = -1e30f;
#pragma unroll
        for (int j = 0; j < EPL; j++) if (lane + 32 * j < E) m = fmaxf(m, v[j]);
        m = warp_max_f32(m);
#pragma unroll
        for (int j = 0; j < EPL; j++)
            if (lane + 32 * j < E) { v[j] = moty_expf(__fsub_rn(v[j], m)); p[lane + 32 * j] = v[j]; }
        __syncwarp();
        const float total = route_seq_sum(p, E);
#pragma unroll
        for (int j = 0; j < EPL; j++)
            if (lane + 32 * j < E) {
                v[j] = __fdiv_rn(v[j], total);
                if (probs_out) probs_out[lane + 32 * j] = v[j];
            }
    }
    float wsum = 0.f;
    float mine = 0.f, mine2 = 0.f;           // lane k keeps weight k (K <= 64: two per lane)
    for (int k = 0; k < K; k++) {
        float bv = -1e30f; int bi = -1;
#pragma unroll
        for (int j = 0; j < EPL; j++) if (v[j] > bv) { bv = v[j]; bi = lane + 32 * j; }
        float gv;
        const int gi = route_pick(bv, bi, gv);
#pragma unroll
        for (int j = 0; j < EPL; j++) if (lane + 32 * j == gi) v[j] = NEG_INF;     // taken: strict > never picks it again
        if (lane == 0) idx_out[k] = gi;
        if ((k & 31) == lane) { if (k < 32) mine = gv; else mine2 = gv; }
        wsum = __fadd_rn(wsum, gv);          // sequential sum in selection order
    }
    if (norm_topk && wsum > 0.f) {
        mine = __fdiv_rn(mine, wsum);
        if (K > 32) mine2 = __fdiv_rn(mine2, wsum);
    }
    if (lane < K) w_out[lane] = mine;
    if (lane + 32 < K) w_out[lane + 32] = mine2;
}

// any E: the row lives in the scratch row; a taken entry is overwritten with -inf there
__device__ __forceinline__ void route_row_warp_mem(const float *__restrict__ lg, int E, int K, float *p, int do_softmax,
                                                   int norm_topk, int lane, int *idx_out, float *w_out,
                                                   float *probs_out) {
    for (int e = lane; e < E; e += 32) p[e] = lg[e];
    __syncwarp();
    if (do_softmax) {
        float m = -1e30f;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, p[e]);
        m = warp_max_f32(m);
        for (int e = lane; e < E; e += 32) p[e] = moty_expf(__fsub_rn(p[e], m));
        __syncwarp();
        const float total = route_seq_sum(p, E);
        __syncwarp();
        for (int e = lane; e < E; e += 32) p[e] = __fdiv_rn(p[e], total);
        __syncwarp();
        if (probs_out)
            for (int e = lane; e < E; e += 32) probs_out[e] = p[e];
    }
    float wsum = 0.f;
    float mine = 0.f, mine2 = 0.f;
    for (int k = 0; k < K; k++) {
        float bv = -1e30f; int bi = -1;
        for (int e = lane; e < E; e += 32) {
            float v = p[e];
            if (v > bv) { bv = v; bi = e; }
        }
        float gv;
        const int gi = route_pick(bv, bi, gv);
        if (gi >= 0 && (gi & 31) == lane) p[gi] = __int_as_float(0xff800000);
        if (lane == 0) idx_out[k] = gi;
        if ((k & 31) == lane) { if (k < 32) mine = gv; else mine2 = gv; }
        wsum = __fadd_rn(wsum, gv);
    }
    if (norm_topk && wsum > 0.f) {
        mine = __fdiv_rn(mine, wsum);
        if (K > 32) mine2 = __fdiv_rn(mine2, wsum);
    }
    if (lane < K) w_out[lane] = mine;
    if (lane + 32 < K) w_out[lane + 32] = mine2;
}

// LFM2's gate (route_sigmoid, nn/moe.c:10-25): probs = 1 / (1 + expf(-logit)); K rounds of "largest probs + bias not
// yet taken" (strict >, ties to the lowest index); the weights are the UNBIASED probabilities of the picks divided by
// their sequential sum when that is positive.  p: 2 E floats of scratch (selection values, then probabilities).
__device__ __forceinline__ void route_row_warp_sigmoid(const float *__restrict__ lg, const float *__restrict__ bias, int E, int K,
                                                       float *p, int lane, int *idx_out, float *w_out) {
    float *pr = p + ((E + 3) & ~3);
    for (int e = lane; e < E; e += 32) {
        const float q = __fdiv_rn(1.f, __fadd_rn(1.f, moty_expf(-lg[e])));
        pr[e] = q;
        p[e] = bias ? __fadd_rn(q, bias[e]) : q;
    }
    __syncwarp();
    float wsum = 0.f, mine = 0.f, mine2 = 0.f;
    for (int k = 0; k < K; k++) {
        float bv = -1e30f; int bi = -1;
        for (int e = lane; e < E; e += 32) {
            const float v = p[e];
            if (v > bv) { bv = v; bi = e; }
        }
        float gv;
        const int gi = route_pick(bv, bi, gv);
        if (gi >= 0 && (gi & 31) == lane) p[gi] = __int_as_float(0xff800000);
        const float q = gi >= 0 ? pr[gi] : 0.f;
        if (lane == 0) idx_out[k] = gi;
        if ((k & 31) == lane) { if (k < 32) mine = q; else mine2 = q; }
        wsum = __fadd_rn(wsum, q);
    }
    if (wsum > 0.f) {
        mine = __fdiv_rn(mine, wsum);
        if (K > 32) mine2 = __fdiv_rn(mine2, wsum);
    }
    if (lane < K) w_out[lane] = mine;
    if (lane + 32 < K) w_out[lane + 32] = mine2;
}

__device__ __forceinline__ void route_row_warp(const float *__restrict__ lg, int E, int K, float *p, int do_softmax,
                                               int norm_topk, int lane, int *idx_out, float *w_out, float *probs_out) {
    if (E <= 64) route_row_warp_reg<2>(lg, E, K, p, do_softmax, norm_topk, lane, idx_out, w_out, probs_out);
    else if (E <= 128) route_row_warp_reg<4>(lg, E, K, p, do_softmax, norm_topk, lane, idx_out, w_out, probs_out);
    else route_row_warp_mem(lg, E, K, p, do_softmax, norm_topk, lane, idx_out, w_out, probs_out);
}
