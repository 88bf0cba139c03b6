// gemv_q8_gateup.cu -- the first half of a dense FFN block for ONE token in one launch:
//     h[i] = act(gate[i] . x) * (up[i] . x)          (engines/qwen.c:520-529 with SiLU, engines/gemma.c:392-398 with tanh-GeLU)
// in place of two products and an element-wise pass.  For the large blocks that the one-launch decode kernel of the
// routed layers does not take (hidden size over 2048 or FFN width over 4096).
//
// A unit is one row index i: the gate row and the up row, 2 x 8 independent 128-bit L1-bypassing loads per lane, dealt
// round-robin to the warps of a persistent grid; the next unit's loads go out before the current result is written.
// Every CTA quantizes the activation row (moty_hw_qrow_i8, hw/hw_quant.h:9-16) into shared memory behind its first
// weight loads.  Same dp4a sums, the same (scale[i] * sx) * (float)dot products (nn/matmul.c:34) and the same
// activation expression as the separate launches: same bits.
// Optionally the residual step and the RMS norm in front of the block ride in the prologue (resnorm.cuh): the row is
// rmsnorm(x + t) * g_x -- or, gemma's sandwich, rmsnorm(x + rmsnorm(t) * g_t) * g_x -- and CTA 0 writes the sum out.
// Limits: rows of 16..4096 int8 values, a multiple of 16; x 16-byte aligned.
#include "kernels.cuh"
#include "resnorm.cuh"

namespace {

constexpr int GLPR = 8;

struct GateUpArgs {
    const int8_t *g, *u; const float *gs, *us;
    const float *x; float *h;
    int O, I16, act;
    const float *t, *g_t, *g_x; float *xout; float eps;    // optional residual + norm prologue (t != nullptr)
};

__global__ void __launch_bounds__(256, 2) q8_gateup_kernel(GateUpArgs a) {
    extern __shared__ int4 smem4[];
    __shared__ float red[8];
    __shared__ double red64[8];
    __shared__ float sx_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int I16 = a.I16, O = a.O, nwarps = gridDim.x * 8;

    int4 wg[GLPR], wu[GLPR];
    float sg = 0.f, su = 0.f;
    auto issue = [&](int o) {
        const int4 *pg = reinterpret_cast<const int4 *>(a.g) + (size_t)o * I16;
        const int4 *pu = reinterpret_cast<const int4 *>(a.u) + (size_t)o * I16;
#pragma unroll
        for (int j = 0; j < GLPR; j++) {
            const int k = j * 32 + lane;
            wg[j] = k < I16 ? ldg_stream16(pg + k) : make_int4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < GLPR; j++) {
            const int k = j * 32 + lane;
            wu[j] = k < I16 ? ldg_stream16(pu + k) : make_int4(0, 0, 0, 0);
        }
        sg = __ldg(a.gs + o); su = __ldg(a.us + o);
    };
    int o = blockIdx.x * 8 + warp;
    pdl_trigger();
    if (o < O) issue(o);                                   // weights only: may run before the previous kernel has finished
    pdl_wait();                                            // the activation row and h from here on

    if (a.t) {   // residual step + norm, then quantize from the f32 copy in shared memory
        float *xf = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(smem4) + I16 * 16);
        const float amax = resnorm_row(a.x, a.t, a.g_t, a.g_x, a.xout, a.eps, I16 * 16, xf, red64, red, blockIdx.x == 0);
        const float sx = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, sx);
        int *xq = reinterpret_cast<int *>(smem4);
        for (int i = threadIdx.x; i < I16 * 4; i += 256) {
            const float4 v = reinterpret_cast<const float4 *>(xf)[i];
            const int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
            const int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
            xq[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        if (threadIdx.x == 0) sx_s = sx;
    } else {   // quantize the row: two passes over x (it sits in L2)
        const int I4 = I16 * 4;
        const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
        float amax = 0.f;
        for (int i = threadIdx.x; i < I4; i += 256) {
            const float4 v = x4[i];
            amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
        }
        amax = warp_max_f32(amax);
        if (lane == 0) red[warp] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
        const float sx = quant_scale(amax, 1e-12f);
        const float inv = __fdiv_rn(1.f, sx);
        int *xq = reinterpret_cast<int *>(smem4);
        for (int i = threadIdx.x; i < I4; i += 256) {
            const float4 v = x4[i];
            const int c0 = quant_code(v.x, inv) & 255, c1 = quant_code(v.y, inv) & 255;
            const int c2 = quant_code(v.z, inv) & 255, c3 = quant_code(v.w, inv) & 255;
            xq[i] = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
        }
        if (threadIdx.x == 0) sx_s = sx;
    }
    __syncthreads();
    const float sx = sx_s;

    while (o < O) {
        int dg = 0, du = 0;
#pragma unroll
        for (int j = 0; j < GLPR; j++) {
            if (j * 32 < I16) {                            // warp-uniform
                int k = j * 32 + lane; k = k < I16 ? k : I16 - 1;      // weights past the row were loaded as zeros
                const int4 xv = smem4[k];
                dg = dp4a4(wg[j], xv, dg);
                du = dp4a4(wu[j], xv, du);
            }
        }
        const float s0 = sg, s1 = su;
        const int row = o;
        o += nwarps;
        if (o < O) issue(o);                               // the next unit's loads go out before this result is written
        dg = warp_sum_i32(dg); du = warp_sum_i32(du);
        if (lane == 0) {
            // (scale * sx) * (float)dot, left to right (nn/matmul.c:34), then the activation (hw/hw_ops.h:19-21, engines/gemma.c:398)
            const float gv = __fmul_rn(__fmul_rn(s0, sx), (float)dg), uv = __fmul_rn(__fmul_rn(s1, sx), (float)du);
            a.h[row] = a.act == MOTY_ACT_SILU ? moty_silu_mul(gv, uv) : moty_gelu_mul(gv, uv);
        }
    }
}

}  // namespace

bool q8_gateup_supported(int I, int D) { return D % 16 == 0 && D >= 16 && D <= 4096 && I >= 1; }

// h[i] = act(gate[i] . x) * (up[i] . x), i < I; gate, up [I][D] int8 with per-row scales; x [D] f32.
int launch_q8_gateup(const int8_t *g, const float *gs, const int8_t *u, const float *us, const float *x, float *h, int I, int D,
                     int act, int sms, cudaStream_t st, const float *t, const float *g_t, const float *g_x, float *xout, float eps) {
    if (!q8_gateup_supported(I, D) || (reinterpret_cast<uintptr_t>(x) & 15))
        return moty_set_error(MOTY_CUDA_EARG, "q8_gateup: %dx%d (rows of 16..4096 bytes, x 16-byte aligned)", I, D);
    if (t && (!g_x || !xout || xout == x)) return moty_set_error(MOTY_CUDA_EARG, "q8_gateup: the residual prologue wants gains and its own output");
    GateUpArgs a;
    a.g = g; a.u = u; a.gs = gs; a.us = us; a.x = x; a.h = h; a.O = I; a.I16 = D / 16; a.act = act;
    a.t = t; a.g_t = t ? g_t : nullptr; a.g_x = g_x; a.xout = xout; a.eps = eps;
    const size_t smem = t ? (size_t)D * 5 : (size_t)D;
    auto k = q8_gateup_kernel;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q8_gateup: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {                          // stored +1 so that zero-init means "nothing cached"
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    if (cached_per_sm[dev] < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "q8_gateup: kernel does not fit (smem %zu)", smem);
    int ctas = sms * cached_per_sm[dev];
    if (ctas > (I + 7) / 8) ctas = (I + 7) / 8;                  // never more warps than units
    CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
    return 0;
}
