// q4r4_stream.cu -- the Q4R4 decode GEMV (1..4 activation rows), persistent and
// software-pipelined.  Same arithmetic as q4r4_small_kernel (q4r4.cu): exact integer
// group sums by dp4a on the split nibbles, and ONE sequential fused-multiply-add
// chain per (row, token) in ascending group order, so the result is bit-identical to
// moty_hw_q4r4_gemm_ref / _gemm4t_ref (hw/hw_q4r4.h:47-84).
//
// Lane layout, chosen per shape by GS (groups side by side in one step):
//   lane = (group-in-step, row-in-unit); a warp unit is 8/GS consecutive 4-row
//   blocks = 32/GS rows; one step covers GS groups of every row of the unit.
//   GS = 1: a lane owns a whole row; its chain needs no shuffle at all (27
//           instructions per 512 bytes) -- for matrices with many rows;
//   GS = 8: a warp owns one block (the layout of q4r4.cu) -- most parallelism, 8
//           chain hops by shuffle per step -- for few, long rows.
// The warps of a persistent grid take units round-robin and see their units as one
// continuous sequence of steps; PF steps are always in flight per warp (a ring of
// registers refilled as soon as a step is consumed), also across unit boundaries.
// With one token the group-of-32 quantizer (moty_hw_quant_g32, hw/hw_q4r4.h:36-45)
// runs inside the kernel: it needs no row-wide reduction.
#include "kernels.cuh"

// unsigned bytes of a times signed bytes of b, accumulated: dp4a.u32.s32
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct Q4StreamArgs {
    const uint8_t *w; const uint16_t *d;
    const float *x;                                            // FUSED: the f32 row
    const int8_t *xq; const float *xs; const int32_t *xsum;    // else: group-quantized rows [S][..]
    const uint8_t *form;                                       // per row, may be null (all token-by-token)
    float *y;
    int S, I, O;
};

template <int NS, int GS, int PF, bool FUSED>
__global__ void __launch_bounds__(256) q4r4_stream_kernel(Q4StreamArgs a) {
    extern __shared__ int4 sm4[];
    constexpr int RL = 32 / GS;                                // rows per unit
    constexpr int BPW = RL / 4;                                // blocks per unit
    const int I = a.I, nb = I / 32, I16 = I / 16, O = a.O;
    int8_t *xq_s = reinterpret_cast<int8_t *>(sm4);
    float *xs_s = reinterpret_cast<float *>(xq_s + (size_t)NS * I);
    int *xsum_s = reinterpret_cast<int *>(xs_s + (size_t)NS * nb);
    __shared__ int form_s[NS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gl = lane / RL, rl = lane % RL, blk_in = rl >> 2, r = rl & 3;
    const int nblk = (O + 3) / 4, nunits = (nblk + BPW - 1) / BPW, nit = (nb + GS - 1) / GS;
    const int nwarps = gridDim.x * 8, gw = blockIdx.x * 8 + warp;
    const int my_units = gw < nunits ? (nunits - gw + nwarps - 1) / nwarps : 0;
    const int total = my_units * nit;                          // steps of this warp (fits an int: < 2^31 / 512 bytes)

    // Loads walk two pointers (codes, scales) that advance by one step; a new unit re-bases them.
    int4 wv[PF]; uint16_t dv[PF];
    int ld_unit = gw, ld_it = 0, ld_j = 0;
    const size_t lane_code = (size_t)gl * 64 + r * 16, lane_scale = (size_t)gl * 4 + r;
    const uint8_t *lp = a.w + ((size_t)(gw * BPW + blk_in) * nb) * 64 + lane_code;
    const uint16_t *dp = a.d + ((size_t)(gw * BPW + blk_in) * nb) * 4 + lane_scale;
    auto load_next = [&](int slot) {
        wv[slot] = make_int4(0, 0, 0, 0); dv[slot] = 0;
        if (ld_j < total) {
            if (ld_it * GS + gl < nb && ld_unit * BPW + blk_in < nblk) {
                wv[slot] = ldg_stream16(lp);
                dv[slot] = __ldg(dp);
            }
            ld_j++; lp += GS * 64; dp += GS * 4;
            if (++ld_it == nit) {
                ld_it = 0; ld_unit += nwarps;
                lp = a.w + ((size_t)(ld_unit * BPW + blk_in) * nb) * 64 + lane_code;
                dp = a.d + ((size_t)(ld_unit * BPW + blk_in) * nb) * 4 + lane_scale;
            }
        }
    };
    pdl_trigger();
#pragma unroll
    for (int u = 0; u < PF; u++) load_next(u);                 // weights only: may overlap the previous kernel
    pdl_wait();

    // ---- activation rows into shared memory ----
    if (FUSED) {
        // one thread per group: eight independent 16-byte loads, a local maximum, no shuffles
        // (a warp-per-group version spent tens of microseconds in dependent shuffles on long rows)
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
            xs_s[g] = s; xsum_s[g] = tot;
        }
        if (threadIdx.x == 0) form_s[0] = 0;
    } else {
        for (int idx = threadIdx.x; idx < NS * I16; idx += 256) {
            int s = idx / I16, k = idx - s * I16;
            sm4[idx] = s < a.S ? reinterpret_cast<const int4 *>(a.xq + (size_t)s * I)[k] : make_int4(0, 0, 0, 0);
        }
        for (int idx = threadIdx.x; idx < NS * nb; idx += 256) {
            int s = idx / nb, g = idx - s * nb;
            xs_s[idx] = s < a.S ? a.xs[(size_t)s * nb + g] : 0.f;
            xsum_s[idx] = s < a.S ? a.xsum[(size_t)s * nb + g] : 0;
        }
        if (threadIdx.x < NS) form_s[threadIdx.x] = (threadIdx.x < a.S && a.form) ? a.form[threadIdx.x] : 0;
    }
    __syncthreads();

    const int prev = (lane + 32 - RL) & 31;                    // lane of the previous group, same row
    float acc[NS];
#pragma unroll
    for (int s = 0; s < NS; s++) acc[s] = 0.f;
    int cur_unit = gw, cur_it = 0;
    for (int j0 = 0; j0 < total; j0 += PF) {
#pragma unroll
        for (int u = 0; u < PF; u++) {
            if (j0 + u >= total) break;                        // warp-uniform
            const int g = cur_it * GS + gl;
            const bool valid = g < nb;
            const int gc = valid ? g : nb - 1;
            const int4 w4 = wv[u];
            const float dd = f16bits_to_f32(dv[u]);
            load_next(u);                                      // refill the slot: PF steps stay in flight
            // low nibbles as they are; high nibbles stay in place (16 x their value) and are read as
            // UNSIGNED bytes by dp4a, the exact factor 16 is shifted out of the sum afterwards
            int4 lo; uint4 hi;
            lo.x = w4.x & 0x0f0f0f0f; hi.x = (unsigned)w4.x & 0xf0f0f0f0u;
            lo.y = w4.y & 0x0f0f0f0f; hi.y = (unsigned)w4.y & 0xf0f0f0f0u;
            lo.z = w4.z & 0x0f0f0f0f; hi.z = (unsigned)w4.z & 0xf0f0f0f0u;
            lo.w = w4.w & 0x0f0f0f0f; hi.w = (unsigned)w4.w & 0xf0f0f0f0u;
            float fs[NS], c0[NS], c1[NS];
#pragma unroll
            for (int s = 0; s < NS; s++) {
                const int4 *xg = reinterpret_cast<const int4 *>(xq_s + (size_t)s * I + gc * 32);
                const int4 x0 = xg[0], x1 = xg[1];
                int sraw = dp4a4(lo, x0, 0);
                int s16 = dp4a_us(hi.x, x1.x, 0);
                s16 = dp4a_us(hi.y, x1.y, s16);
                s16 = dp4a_us(hi.z, x1.z, s16);
                s16 = dp4a_us(hi.w, x1.w, s16);
                sraw += s16 >> 4;
                const float xsc = xs_s[s * nb + gc];
                const int xsm = xsum_s[s * nb + gc];
                c0[s] = __fmul_rn(dd, xsc);
                if (form_s[s]) {                               // 4-token tile formula (hw/hw_q4r4.h:78-81)
                    fs[s] = (float)sraw;
                    c1[s] = __fmul_rn(__fmul_rn(8.f, (float)xsm), xsc);
                } else {                                       // token-by-token formula (hw/hw_q4r4.h:58-59)
                    fs[s] = (float)(sraw - 8 * xsm);
                    c1[s] = 0.f;
                }
            }
            if (GS == 1) {                                     // the lane owns the row: plain sequential chain
#pragma unroll
                for (int s = 0; s < NS; s++) {
                    if (valid) {
                        float t = fmaf(fs[s], c0[s], acc[s]);
                        if (form_s[s]) t = fmaf(-dd, c1[s], t);
                        acc[s] = t;
                    }
                }
            } else {
#pragma unroll
                for (int jj = 0; jj < GS; jj++) {
#pragma unroll
                    for (int s = 0; s < NS; s++) {
                        float in = __shfl_sync(0xffffffffu, acc[s], prev);
                        if (gl == jj) {
                            float t = in;
                            if (valid) {
                                t = fmaf(fs[s], c0[s], in);
                                if (form_s[s]) t = fmaf(-dd, c1[s], t);
                            }
                            acc[s] = t;
                        }
                    }
                }
            }
            if (++cur_it == nit) {                             // unit finished: the lanes of the last group hold the rows
                if (gl == GS - 1) {
                    int o = (cur_unit * BPW + blk_in) * 4 + r;
                    if (o < O) {
#pragma unroll
                        for (int s = 0; s < NS; s++)
                            if (s < a.S) a.y[(size_t)s * O + o] = acc[s];
                    }
                }
#pragma unroll
                for (int s = 0; s < NS; s++) acc[s] = 0.f;
                cur_it = 0; cur_unit += nwarps;
            }
        }
    }
}

template <int NS, int GS, int PF, bool FUSED>
static int launch_q4s_t(const Q4StreamArgs &a, int sms, cudaStream_t st) {
    int nb = a.I / 32;
    size_t smem = (size_t)NS * a.I + (size_t)NS * nb * 8;
    auto k = q4r4_stream_kernel<NS, GS, PF, FUSED>;
    static size_t cached_smem[MOTY_MAX_DEV];
    static int cached_per_sm[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q4r4_stream: device %d", dev);
    if (smem + 1 != cached_smem[dev]) {
        if (smem > 48 * 1024) CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&cached_per_sm[dev], k, 256, smem));
        cached_smem[dev] = smem + 1;
    }
    int per_sm = cached_per_sm[dev];
    if (per_sm < 1) return moty_set_error(MOTY_CUDA_ELIMIT, "q4r4_stream: kernel does not fit (smem %zu)", smem);
    int nunits = ((a.O + 3) / 4 + (8 / GS) - 1) / (8 / GS);
    int ctas = sms * per_sm;
    if (ctas > (nunits + 7) / 8) ctas = (nunits + 7) / 8;
    CK(moty_launch_pdl(k, dim3(ctas), dim3(256), smem, st, a));
    return 0;
}

template <int NS, bool FUSED>
static int launch_q4s_gs(const Q4StreamArgs &a, int sms, cudaStream_t st) {
    // the fewest groups side by side that still give every SM about a dozen warps of work
    const long long nblk = (a.O + 3) / 4, want = (long long)sms * 12;
    if (nblk / 8 >= want) return launch_q4s_t<NS, 1, (NS <= 2 ? 8 : 4), FUSED>(a, sms, st);
    if (nblk / 4 >= want) return launch_q4s_t<NS, 2, 4, FUSED>(a, sms, st);
    if (nblk / 2 >= want) return launch_q4s_t<NS, 4, 4, FUSED>(a, sms, st);
    return launch_q4s_t<NS, 8, (NS <= 2 ? 8 : 4), FUSED>(a, sms, st);
}

// x: the f32 row when S == 1 (quantized in the kernel); xq/xs/xsum: the quantized rows otherwise
int launch_q4r4_stream(const uint8_t *w, const uint16_t *d, const float *x, const int8_t *xq, const float *xs,
                       const int32_t *xsum, const uint8_t *form, float *y, int S, int I, int O, int sms, cudaStream_t st) {
    if (I % 32 != 0 || I <= 0 || I > MOTY_QROW_MAX || S < 1 || S > 4) return moty_set_error(MOTY_CUDA_EARG, "q4r4_stream: S=%d I=%d", S, I);
    if (O <= 0) return 0;
    Q4StreamArgs a;
    a.w = w; a.d = d; a.x = x; a.xq = xq; a.xs = xs; a.xsum = xsum; a.form = form; a.y = y; a.S = S; a.I = I; a.O = O;
    if (S == 1 && x && q4r4_gemv1_supported(I, O, sms)) return launch_q4r4_gemv1(w, d, x, y, I, O, sms, st);   // many rows: lane = row
    if (S == 1 && x) return launch_q4s_gs<1, true>(a, sms, st);
    if (S == 1) return launch_q4s_gs<1, false>(a, sms, st);
    if (S == 2) return launch_q4s_gs<2, false>(a, sms, st);
    return launch_q4s_gs<4, false>(a, sms, st);
}
