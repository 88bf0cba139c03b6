// q4_decode.cuh -- pieces shared by the Q4R4 decode kernels of the MoE block
// (moe_decode_q4.cu, moe_decode_fused_q4.cu): the group-of-32 activation quantizer and one
// 512-byte step of a 4-row block with its sequential chain hop.
//
// Layout of a step: a warp owns one 4-row block, lane = (group-in-step << 2) | row, 512
// contiguous bytes of codes per step, the running sum of a row hops from the lane of group g to
// the lane of group g+1 by shuffle (ascending group order, one fused multiply-add per group:
// hw/hw_q4r4.h:47-63).
#pragma once
#include "common.cuh"

// One group of 32 floats at src -> 32 codes at dst8, its scale and the sum of its codes
// (moty_hw_quant_g32, hw/hw_q4r4.h:36-45).  COHERENT: read through L2, for floats that other
// CTAs of the same launch wrote.
template <bool COHERENT>
__device__ __forceinline__ void quant_group32(const float *src, int8_t *dst8, float &s_out, int &sum_out) {
    const float4 *p = reinterpret_cast<const float4 *>(src);
    float4 v[8];
#pragma unroll
    for (int k = 0; k < 8; k++) v[k] = COHERENT ? __ldcg(p + k) : p[k];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++)
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w))));
    const float s = quant_scale(amax, 1e-30f);
    const float inv = __fdiv_rn(1.f, s);
    int tot = 0;
    int *dst = reinterpret_cast<int *>(dst8);
#pragma unroll
    for (int k = 0; k < 8; k++) {
        int c0 = quant_code(v[k].x, inv), c1 = quant_code(v[k].y, inv);
        int c2 = quant_code(v[k].z, inv), c3 = quant_code(v[k].w, inv);
        tot += c0 + c1 + c2 + c3;
        dst[k] = (c0 & 255) | ((c1 & 255) << 8) | ((c2 & 255) << 16) | ((c3 & 255) << 24);
    }
    s_out = s; sum_out = tot;
}

// ngroups groups at src, one thread per group, threads tid, tid + nthreads, ...
__device__ __forceinline__ void quant_groups(const float *src, int ngroups, int8_t *xq, float *xs, int *xsum,
                                             int tid, int nthreads) {
    for (int g = tid; g < ngroups; g += nthreads)
        quant_group32<false>(src + (size_t)g * 32, xq + (size_t)g * 32, xs[g], xsum[g]);
}

// one 512-byte step of one block: the lane's (row, group) integer sum and its chain factor
__device__ __forceinline__ void q4_step_terms(const int4 &w4, uint16_t dbits, const int8_t *xq_s, const float *xs_s,
                                              const int *xsum_s, int gc, float &fs, float &c0) {
    int4 lo, hi;
    lo.x = w4.x & 0x0f0f0f0f; hi.x = (w4.x >> 4) & 0x0f0f0f0f;
    lo.y = w4.y & 0x0f0f0f0f; hi.y = (w4.y >> 4) & 0x0f0f0f0f;
    lo.z = w4.z & 0x0f0f0f0f; hi.z = (w4.z >> 4) & 0x0f0f0f0f;
    lo.w = w4.w & 0x0f0f0f0f; hi.w = (w4.w >> 4) & 0x0f0f0f0f;
    const int4 *xg = reinterpret_cast<const int4 *>(xq_s + (size_t)gc * 32);
    int sraw = dp4a4(lo, xg[0], 0);
    sraw = dp4a4(hi, xg[1], sraw);
    fs = (float)(sraw - 8 * xsum_s[gc]);
    c0 = __fmul_rn(f16bits_to_f32(dbits), xs_s[gc]);
}

// the chain hop of one step: 8 groups side by side, ascending
__device__ __forceinline__ float q4_chain(float acc, float fs, float c0, bool valid, int gl, int prev) {
#pragma unroll
    for (int jj = 0; jj < 8; jj++) {
        float in = __shfl_sync(0xffffffffu, acc, prev);
        if (gl == jj) acc = valid ? fmaf(fs, c0, in) : in;
    }
    return acc;
}
