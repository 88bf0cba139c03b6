// q4r4_gemv2.cu -- the Q4R4 decode GEMV for matrices with too few rows to give every SM
// a dozen warps of whole rows (FFN projections): two phases.
//
// The reference (moty_hw_q4r4_gemm_ref, hw/hw_q4r4.h:47-63) has two layers of arithmetic: per
// group of 32 weights an exact integer sum, and across the groups of a row ONE sequential f32
// chain, acc = fma((float)(sum - 8 * xsum), d * xs, acc) in ascending group order.  The integer
// layer is where the bytes are and has no order; the chain must stay sequential but needs only
// the two f32 factors of each fused multiply-add.  So:
//   phase 1  every (block, group) cell of 64 bytes is independent.  A CTA owns a slab of 32
//            consecutive groups and a share of the 4-row blocks: it group-quantizes just those
//            1024 activations (moty_hw_quant_g32, hw/hw_q4r4.h:36-45), every lane keeps the codes
//            of the 4 groups it will ever meet in registers, and the warps stream 2 KB pieces
//            (one block x slab) in coalesced 512-byte loads, 4 lanes per cell, one per row.
//            Both factors, (float)(sum - 8 * xsum) and d * xs, go to a scratch table laid out for
//            phase 2, ab[32-row band][group pair][32 rows][a, b, a', b'] (O x I/32 x 8 bytes: a
//            few MB, it stays in L2);
//   phase 2  a CTA is one warp and takes a band of 32 rows: the band's table is one contiguous
//            run that arrives in shared memory through bulk asynchronous copies of 8 KB, each
//            with its own mbarrier (bounded waits), and the warp, lane = row, runs the chain as
//            the pieces land: one conflict-free 16-byte shared load and two fmas per group pair.
// Phase 1 runs at memory speed whatever the shape (a 3840 x 15360 matrix has 120 warps' worth of
// rows but 1.8 M cells); phase 2 costs a few microseconds of dependent arithmetic.
// Same bits as the one-phase kernels (q4r4_gemv1.cu, q4r4_stream.cu).  Q8R4 matrices (the int8 sibling, 128 bytes per
// cell, no offset term) take the same two phases for every shape.
#include "kernels.cuh"
#include <string.h>

namespace {

struct Q4G2Args {
    const uint8_t *w; const uint16_t *d;
    const float *x; float *y;
    float *ab;                       // [bands][(nb + 1) / 2][32][4]
    int I, O;
    int cps;                         // phase 1: CTAs per slab
    int *err;                        // phase 2: set when a bounded wait expired
    // WF_I4G (i4g_g2_sums_kernel): f32 group scales [O][nb], the row's int8 codes and its scale from qrow_i8
    const float *gscale; const int8_t *xi; const float *sx;
};

__device__ __forceinline__ int dp4a_us2(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Phase 1 works in warp steps of 512 bytes, four steps to a stage.  Q4R4: a cell is 64 bytes, 4 lanes per cell (one
// per row), 8 cells per step, so a stage is one block x a slab of 32 groups.  Q8R4 (Q8 = true; hw/hw_q4r4.h:92-130:
// 128 bytes per cell = 4 rows x 32 signed codes, no offset term): 8 lanes per cell (two per row, 16 codes each, sums
// joined by one shuffle), 4 cells per step, a slab of 16 groups.
constexpr int G2_NST = 4;            // stages in a warp's ring: 3 on their way while one is consumed
constexpr int G2_STAGE = 2048 + 512; // codes as they lie in memory, then one 4-byte slot per lane and step for its f16 scale
constexpr size_t G2_RING = (size_t)8 * G2_NST * G2_STAGE;

template <bool Q8>
__global__ void __launch_bounds__(256, 2) q4r4_g2_sums_kernel(Q4G2Args a) {
    constexpr int SLAB = Q8 ? 16 : 32;                                  // groups per slab
    constexpr int LPC = Q8 ? 8 : 4, CPS = 32 / LPC;                     // lanes per cell, cells per step
    constexpr int CELL = Q8 ? 128 : 64;
    constexpr int XW = Q8 ? 4 : 8;                                      // words of activation codes a lane needs per group
    extern __shared__ __align__(16) unsigned char ring[];               // [warp][stage][G2_STAGE]
    __shared__ __align__(16) int xq_s[32 * 8];                          // the slab's codes, 4 per word
    __shared__ int x8_s[32];                                            // 8 * code sum per group (Q4R4's offset term)
    __shared__ float xs_s[32];                                          // group scales
    const int nb = a.I / 32, nblk = (a.O + 3) / 4;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int slab = blockIdx.x / a.cps, j = blockIdx.x - slab * a.cps;
    const int g_base = slab * SLAB;
    const int ng = nb - g_base < SLAB ? nb - g_base : SLAB;
    // the lane's cell in step q: group cl + CPS q; its row; (Q8R4) which 16 of the row's 32 codes
    const int cl = lane / LPC, r = Q8 ? (lane >> 1) & 3 : lane & 3, half = Q8 ? lane & 1 : 0;
    const int bstride = a.cps * 8, blk0 = j * 8 + warp;
    const int nmine = blk0 < nblk ? (nblk - 1 - blk0) / bstride + 1 : 0;  // blocks this warp takes: blk0 + i * bstride

    // Every lane copies exactly the bytes it will consume (its 16 bytes of codes per step, the aligned 4 bytes that
    // hold its f16 scale), so a stage needs no barrier: cp.async.wait_group orders a thread's own copies.
    unsigned char *my = ring + (size_t)warp * G2_NST * G2_STAGE + lane * 16;
    const uint8_t *lane_w = a.w + (size_t)g_base * CELL + lane * 16;    // a step is 512 consecutive bytes
    const uint8_t *lane_d = reinterpret_cast<const uint8_t *>(a.d) + (((size_t)g_base + cl) * 4 + (r & 2)) * 2;
    auto issue = [&](int i) {
        if (i < nmine) {
            const size_t b = (size_t)(blk0 + i * bstride);
            const uint8_t *pw = lane_w + b * nb * CELL, *pd = lane_d + b * nb * 8;
            unsigned char *st = my + (i % G2_NST) * G2_STAGE;
#pragma unroll
            for (int q = 0; q < 4; q++)
                if (cl + CPS * q < ng) {
                    cp_async16(st + q * 512, pw + q * 512);
                    cp_async4(st + 2048 + q * 128 - lane * 12, pd + q * CPS * 8);   // slot q * 128 + lane * 4
                }
        }
        cp_async_commit();
    };
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < G2_NST - 1; i++) issue(i);                      // weights only: may overlap the previous kernel
    pdl_wait();

    {   // the slab of the activation row: 8 threads per group, 4 values each
        const int g = t >> 3, part = t & 7;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (g < ng) v = reinterpret_cast<const float4 *>(a.x + ((size_t)g_base + g) * 32)[part];
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float s = quant_scale(amax, 1e-30f);
        const float inv = __fdiv_rn(1.f, s);
        const int c0 = quant_code(v.x, inv), c1 = quant_code(v.y, inv);
        const int c2 = quant_code(v.z, inv), c3 = quant_code(v.w, inv);
        int tot = c0 + c1 + c2 + c3;
        tot += __shfl_xor_sync(0xffffffffu, tot, 1);
        tot += __shfl_xor_sync(0xffffffffu, tot, 2);
        tot += __shfl_xor_sync(0xffffffffu, tot, 4);
        xq_s[t] = (c0 & 255) | ((c1 & 255) << 8) | ((c2 & 255) << 16) | ((c3 & 255) << 24);
        if (part == 0) {
            x8_s[g] = Q8 ? 0 : 8 * tot;
            xs_s[g] = s;
        }
    }
    __syncthreads();
    // the lane meets 4 groups only: their codes, offsets and scales stay in registers
    int xr[4][XW], x8[4]; float xsr[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const int gq = cl + CPS * q;
        const int4 *p = reinterpret_cast<const int4 *>(xq_s + gq * 8 + half * 4);
        const int4 lo = p[0];
        xr[q][0] = lo.x; xr[q][1] = lo.y; xr[q][2] = lo.z; xr[q][3] = lo.w;
        if (!Q8) {
            const int4 hi = p[1];
            xr[q][XW - 4] = hi.x; xr[q][XW - 3] = hi.y; xr[q][XW - 2] = hi.z; xr[q][XW - 1] = hi.w;
        }
        x8[q] = x8_s[gq];
        xsr[q] = xs_s[gq];
    }
    // ab[band][pair][32][4]: the lane's row inside its band depends on the block only
    const int nb2 = (nb + 1) / 2;
    for (int i = 0; i < nmine; i++) {
        issue(i + G2_NST - 1);
        cp_async_wait<G2_NST - 1>();                                     // stage i has landed
        const int b = blk0 + i * bstride;
        const unsigned char *st = my + (i % G2_NST) * G2_STAGE;
        float *out = a.ab + (((size_t)(b >> 3) * nb2 + (g_base >> 1) + (cl >> 1)) * 32 + (b & 7) * 4 + r) * 4 + (cl & 1) * 2;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int4 w4 = *reinterpret_cast<const int4 *>(st + q * 512);
            const uint16_t dq = *reinterpret_cast<const uint16_t *>(st + 2048 + q * 128 - lane * 12 + (r & 1) * 2);
            int sraw;
            if (Q8) {                                                    // 16 of the row's 32 products, the other lane has the rest
                sraw = __dp4a(w4.x, xr[q][0], 0);
                sraw = __dp4a(w4.y, xr[q][1], sraw);
                sraw = __dp4a(w4.z, xr[q][2], sraw);
                sraw = __dp4a(w4.w, xr[q][3], sraw);
                sraw += __shfl_xor_sync(0xffffffffu, sraw, 1);
            } else {
                // low nibbles as they are; high nibbles stay in place (16 x their value), are read as UNSIGNED bytes by
                // dp4a and the exact factor 16 is shifted out of the sum afterwards
                sraw = __dp4a(w4.x & 0x0f0f0f0f, xr[q][0], 0);
                sraw = __dp4a(w4.y & 0x0f0f0f0f, xr[q][1], sraw);
                sraw = __dp4a(w4.z & 0x0f0f0f0f, xr[q][2], sraw);
                sraw = __dp4a(w4.w & 0x0f0f0f0f, xr[q][3], sraw);
                int s16 = dp4a_us2((unsigned)w4.x & 0xf0f0f0f0u, xr[q][XW - 4], 0);
                s16 = dp4a_us2((unsigned)w4.y & 0xf0f0f0f0u, xr[q][XW - 3], s16);
                s16 = dp4a_us2((unsigned)w4.z & 0xf0f0f0f0u, xr[q][XW - 2], s16);
                s16 = dp4a_us2((unsigned)w4.w & 0xf0f0f0f0u, xr[q][XW - 1], s16);
                sraw += s16 >> 4;
            }
            // the two factors of the chain's fma (hw/hw_q4r4.h:58-59, :103-104)
            if (cl + CPS * q < ng && half == 0)
                *reinterpret_cast<float2 *>(out + q * (CPS / 2) * 128) =
                    make_float2((float)(sraw - x8[q]), __fmul_rn(f16bits_to_f32(dq), xsr[q]));
        }
    }
    cp_async_wait<0>();
}

// ---- phase 1 for WF_I4G (grouped int4, rows of I/2 bytes, f32 group scales [O][nb]; nn/matmul.c:164-197 with
// IDOT4=1, hw/hw_quant.h:35-50): a CTA owns a slab of 32 groups = 512 consecutive bytes of every row, lane = group.
// The activation row was quantized per ROW by qrow_i8; the lane keeps its group's codes, split into even and odd
// elements (a byte holds the even element in its low nibble), in registers.  A warp step is four rows: four
// coalesced 512-byte loads of codes and four 128-byte loads of scales, two register buffers alternate.
// Factors of the chain's fma: (float)(sum(nibble * x) - 8 * sum(x)) and scl[g]; the chain kernel multiplies by sx.
constexpr int G2I_R = 4;
__global__ void __launch_bounds__(256, 2) i4g_g2_sums_kernel(Q4G2Args a) {
    const int nb = a.I / 32, O = a.O;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slab = blockIdx.x / a.cps, j = blockIdx.x - slab * a.cps;
    const int g = slab * 32 + lane;
    const bool gin = g < nb;
    const int gc = gin ? g : nb - 1;                                    // groups past the row: a valid address, nothing stored
    const int rstride = a.cps * 8 * G2I_R;
    int row = (j * 8 + warp) * G2I_R;
    const uint8_t *wp = a.w + (size_t)gc * 16;
    const float *sp = a.gscale + gc;
    const size_t rb = (size_t)a.I / 2;

    uint4 wA[G2I_R], wB[G2I_R]; float cA[G2I_R], cB[G2I_R];
    auto load = [&](uint4 (&wv)[G2I_R], float (&cv)[G2I_R], int r0) {
#pragma unroll
        for (int u = 0; u < G2I_R; u++) {
            const int r = r0 + u < O ? r0 + u : O - 1;
            const int4 t = ldg_stream16(wp + (size_t)r * rb);
            wv[u] = make_uint4((unsigned)t.x, (unsigned)t.y, (unsigned)t.z, (unsigned)t.w);
            cv[u] = __ldg(sp + (size_t)r * nb);
        }
    };
    pdl_trigger();
    if (row < O) load(wA, cA, row);                                     // weights only: may overlap the previous kernel
    pdl_wait();                                                         // the codes come from the quantizer launch
    int xe[4], xo[4], x8;
    {
        const int4 *src = reinterpret_cast<const int4 *>(a.xi + (size_t)gc * 32);
        const int4 x0 = src[0], x1 = src[1];
        xe[0] = __byte_perm(x0.x, x0.y, 0x6420); xo[0] = __byte_perm(x0.x, x0.y, 0x7531);
        xe[1] = __byte_perm(x0.z, x0.w, 0x6420); xo[1] = __byte_perm(x0.z, x0.w, 0x7531);
        xe[2] = __byte_perm(x1.x, x1.y, 0x6420); xo[2] = __byte_perm(x1.x, x1.y, 0x7531);
        xe[3] = __byte_perm(x1.z, x1.w, 0x6420); xo[3] = __byte_perm(x1.z, x1.w, 0x7531);
        int sum = 0;
#pragma unroll
        for (int k = 0; k < 4; k++) { sum = __dp4a(xe[k], 0x01010101, sum); sum = __dp4a(xo[k], 0x01010101, sum); }
        x8 = 8 * sum;
    }
    const int nb2 = (nb + 1) / 2;
    float *out0 = a.ab + ((size_t)(g >> 1) * 32) * 4 + (g & 1) * 2;      // + (band * nb2 * 32 + row in band) * 4
    auto consume = [&](const uint4 (&cur)[G2I_R], const float (&ccur)[G2I_R], uint4 (&nxt)[G2I_R], float (&cnxt)[G2I_R]) {
        const int r0 = row;
        row += rstride;
        if (row < O) load(nxt, cnxt, row);
#pragma unroll
        for (int u = 0; u < G2I_R; u++) {
            const int r = r0 + u;
            const uint4 w = cur[u];
            int d = __dp4a((int)(w.x & 0x0f0f0f0fu), xe[0], -x8);
            d = __dp4a((int)(w.y & 0x0f0f0f0fu), xe[1], d);
            d = __dp4a((int)(w.z & 0x0f0f0f0fu), xe[2], d);
            d = __dp4a((int)(w.w & 0x0f0f0f0fu), xe[3], d);
            d = __dp4a((int)((w.x >> 4) & 0x0f0f0f0fu), xo[0], d);
            d = __dp4a((int)((w.y >> 4) & 0x0f0f0f0fu), xo[1], d);
            d = __dp4a((int)((w.z >> 4) & 0x0f0f0f0fu), xo[2], d);
            d = __dp4a((int)((w.w >> 4) & 0x0f0f0f0fu), xo[3], d);
            if (gin && r < O)
                *reinterpret_cast<float2 *>(out0 + ((size_t)(r >> 5) * nb2 * 32 + (r & 31)) * 4) = make_float2((float)d, ccur[u]);
        }
    };
    while (row < O) {
        consume(wA, cA, wB, cB);
        if (row >= O) break;
        consume(wB, cB, wA, cA);
    }
}

// ---- phase 2: one warp per CTA, a band of 32 rows, lane = row (hw/hw_q4r4.h:58-59) ----
constexpr int G2_PIECE = 16;                      // group pairs per bulk copy: 8 KB
constexpr unsigned G2_WAIT_LIMIT = 1u << 26;

__device__ __forceinline__ unsigned g2_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool g2_wait(unsigned long long *bar, unsigned parity) {
    return moty_mbar_wait_bounded(g2_smem(bar), parity, G2_WAIT_LIMIT);
}

__global__ void __launch_bounds__(32) q4r4_g2_chain_kernel(Q4G2Args a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int nb = a.I / 32, nb2 = (nb + 1) / 2, O = a.O;
    const int lane = threadIdx.x, band = blockIdx.x;
    const int npieces = (nb2 + G2_PIECE - 1) / G2_PIECE;
    float4 *ab_s = reinterpret_cast<float4 *>(smem);                     // [nb2][32]
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(smem + (size_t)nb2 * 512);
    if (lane == 0) {
        for (int p = 0; p < npieces; p++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(g2_smem(&bars[p])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    pdl_trigger();
    pdl_wait();                                                          // the table comes from phase 1
    if (lane == 0) {
        const float4 *src = reinterpret_cast<const float4 *>(a.ab) + (size_t)band * nb2 * 32;
        for (int p = 0; p < npieces; p++) {
            const int np = nb2 - p * G2_PIECE < G2_PIECE ? nb2 - p * G2_PIECE : G2_PIECE;
            const unsigned bytes = (unsigned)np * 512u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(g2_smem(&bars[p])), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(g2_smem(ab_s + (size_t)p * G2_PIECE * 32)), "l"(src + (size_t)p * G2_PIECE * 32), "r"(bytes),
                           "r"(g2_smem(&bars[p])) : "memory");
        }
    }
    const int nfull = nb / 2;                                            // pairs with both groups
    float acc = 0.f;
    bool ok = true;
    for (int p = 0; p < npieces && ok; p++) {
        ok = g2_wait(&bars[p], 0);
        if (!ok) break;
        const float4 *v = ab_s + (size_t)p * G2_PIECE * 32 + lane;
        const int n = nfull - p * G2_PIECE < G2_PIECE ? nfull - p * G2_PIECE : G2_PIECE;
        if (n == G2_PIECE) {
#pragma unroll
            for (int h = 0; h < G2_PIECE; h += 8) {                       // 8 loads on their way before the first fma needs one
                float4 f[8];
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = v[(h + i) * 32];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    acc = fmaf(f[i].x, f[i].y, acc);
                    acc = fmaf(f[i].z, f[i].w, acc);
                }
            }
        } else {
            for (int i = 0; i < n; i++) {
                const float4 f = v[i * 32];
                acc = fmaf(f.x, f.y, acc);
                acc = fmaf(f.z, f.w, acc);
            }
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
        // a bounded wait expired: copies may still be in flight towards this CTA's memory; give them time, report
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        if (lane == 0) atomicExch(a.err, 1);
        return;
    }
    if (nb & 1) {                                                        // an odd group count: the last pair is half full
        const float4 f = ab_s[(size_t)nfull * 32 + lane];
        acc = fmaf(f.x, f.y, acc);
    }
    if (a.sx) acc = __fmul_rn(*a.sx, acc);                              // WF_I4G: sx * dot (nn/matmul.c:157)
    if (band * 32 + lane < O) a.y[band * 32 + lane] = acc;
}

}  // namespace

// Q4R4: worth two launches when there are enough cells to occupy the machine and few enough rows that the lane-per-row
// kernels starve (3840 x 15360: 9.7 us against 31.6 us of the bulk-fed kernel, 15360 x 3840: 9.1 against 15.2,
// 5120 x 13824: 10.5 against 28.5; from 32000 x 4096 on the one-phase kernels are level or ahead: 19.7 against
// 18.5 us, and the vocabulary matrix 151936 x 1024 takes 20.5 against 17.2 us of q4r4_gemv1_kernel).
// Q8R4 has no one-phase decode kernel: every matrix comes here.
bool q4r4_gemv2_supported(int I, int O, int q8, int sms) {
    if (I % 32 != 0 || I <= 0 || I > MOTY_QROW_MAX || O <= 0) return false;
    if (q8) return true;
    const int nbands = (O + 31) / 32;
    // from 60 k cells up (2048 x 4096): measured inside a Qwen3-30B-A3B-shaped decode step, where the projections
    // around the attention are 5120 x 2048 and 2048 x 4096 -- 2.71 -> 2.38 ms per token against the one-launch
    // streaming kernel, although timed alone in a loop of its own the two launches are the slower ones at that size
    // (9.2 against 5.7 us on 5120 x 2048): their first phase streams weights before its dependency wait
    return nbands < sms * 6 && (long long)((O + 3) / 4) * (I / 32) >= 60000;
}

// WF_I4G through the two phases: xi/sx are the row quantized by qrow_i8 (same stream, just before)
int launch_i4g_gemv2(const uint8_t *w4, const float *gscale, const int8_t *xi, const float *sx, float *y, float *ab,
                     int *err, int I, int O, int sms, cudaStream_t st) {
    if (I % 32 != 0 || I <= 0 || I > MOTY_QROW_MAX || O <= 0) return moty_set_error(MOTY_CUDA_EARG, "i4g_gemv2: I=%d O=%d", I, O);
    Q4G2Args a; memset(&a, 0, sizeof a);
    a.w = w4; a.gscale = gscale; a.xi = xi; a.sx = sx; a.y = y; a.ab = ab; a.err = err; a.I = I; a.O = O;
    const int nb = I / 32, nslab = (nb + 31) / 32;
    int cps = sms * 2 / nslab;
    if (cps < 1) cps = 1;
    if (cps > (O + 8 * G2I_R - 1) / (8 * G2I_R)) cps = (O + 8 * G2I_R - 1) / (8 * G2I_R);
    a.cps = cps;
    const int nb2 = (nb + 1) / 2;
    const size_t smem2 = (size_t)nb2 * 512 + (size_t)((nb2 + G2_PIECE - 1) / G2_PIECE) * 8;
    static bool attr_set[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "i4g_gemv2: device %d", dev);
    if (!attr_set[dev]) {
        CK(cudaFuncSetAttribute(q4r4_g2_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                MOTY_QROW_MAX / 64 * 512 + 16 * 8));
        attr_set[dev] = true;
    }
    CK(moty_launch_pdl(i4g_g2_sums_kernel, dim3((unsigned)(cps * nslab)), dim3(256), (size_t)0, st, a));
    CK(moty_launch_pdl(q4r4_g2_chain_kernel, dim3((unsigned)((O + 31) / 32)), dim3(32), smem2, st, a));
    return 0;
}

size_t q4r4_gemv2_scratch_bytes(int I, int O) { return (size_t)((O + 31) / 32) * ((I / 32 + 1) / 2) * 32 * 16; }

// x: 16-byte aligned; ab: q4r4_gemv2_scratch_bytes(I, O), 128-byte aligned; err: set when a bounded wait expired;
// q8 != 0: w holds Q8R4 codes
int launch_q4r4_gemv2(const uint8_t *w, const uint16_t *d, const float *x, float *y, float *ab, int *err,
                      int I, int O, int q8, int sms, cudaStream_t st) {
    if (!q4r4_gemv2_supported(I, O, q8, sms)) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv2: I=%d O=%d", I, O);
    Q4G2Args a; memset(&a, 0, sizeof a);
    a.w = w; a.d = d; a.x = x; a.y = y; a.ab = ab; a.err = err; a.I = I; a.O = O;
    const int nb = I / 32, slab = q8 ? 16 : 32, nslab = (nb + slab - 1) / slab, nblk = (O + 3) / 4;
    int cps = sms * 2 / nslab;
    if (cps < 1) cps = 1;
    if (cps > (nblk + 7) / 8) cps = (nblk + 7) / 8;
    a.cps = cps;
    const int nb2 = (nb + 1) / 2;
    const size_t smem2 = (size_t)nb2 * 512 + (size_t)((nb2 + G2_PIECE - 1) / G2_PIECE) * 8;   // at most 256 pairs: 128 KB
    static bool attr_set[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv2: device %d", dev);
    if (!attr_set[dev]) {
        CK(cudaFuncSetAttribute(q4r4_g2_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                MOTY_QROW_MAX / 64 * 512 + 16 * 8));
        CK(cudaFuncSetAttribute(q4r4_g2_sums_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G2_RING));
        CK(cudaFuncSetAttribute(q4r4_g2_sums_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G2_RING));
        attr_set[dev] = true;
    }
    if (q8) CK(moty_launch_pdl(q4r4_g2_sums_kernel<true>, dim3((unsigned)(cps * nslab)), dim3(256), G2_RING, st, a));
    else CK(moty_launch_pdl(q4r4_g2_sums_kernel<false>, dim3((unsigned)(cps * nslab)), dim3(256), G2_RING, st, a));
    CK(moty_launch_pdl(q4r4_g2_chain_kernel, dim3((unsigned)((O + 31) / 32)), dim3(32), smem2, st, a));
    return 0;
}
