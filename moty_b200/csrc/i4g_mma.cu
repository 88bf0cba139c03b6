// i4g_mma.cu -- WF_I4G weights (grouped int4, group 32, f32 group scales, row-major nibbles) x a batch of
// row-quantized int8 activations: the integer path of moty_matmul_i4_grouped_s (nn/matmul.c:164-197 with IDOT4=1;
// moty_hw_dot_i4g8p, hw/hw_quant.h:35-50) for batches, on the tensor cores.
//
// Per (row, token) the reference forms, for every group of 32 weights, the exact integer d = sum((nibble - 8) * x)
// and adds ONE f32 term per group in ascending group order, acc = fma(scl[g], (float)d, acc), then returns sx * acc.
// The integer sum has no order, so it is one mma.sync.m16n8k32 (u8 nibble codes x s8 activation codes -> s32) per group
// and 16 rows x 8 tokens; the chain stays in registers, as in q4r4_mma.cu:
//   * the accumulator INPUT of the MMA is 0x4B400000 - 8 * (sum of the token's codes in the group), a per-(group, token)
//     record: the instruction returns the bit pattern of the float 1.5 * 2^23 + d, and one exact FADD leaves (float)d;
//   * FADD and FFMA run as packed add / fma.rn.f32x2, two tokens per instruction (same rounding per lane).
// Fragment fit: a row's group is 16 bytes, byte b = element 2b | element 2b+1 << 4.  Word t of it holds elements
// 8t .. 8t+7: its low nibbles (the even ones) go to fragment slots k = 4t .. 4t+3, its high nibbles (the odd ones) to
// k = 16+4t .. -- a permutation of the group, harmless for an integer sum as long as the activations follow it: a thread
// loads the 8 codes 8t .. 8t+7 of its token with one 64-bit load and splits them into evens and odds with two PRMTs.
//
// A CTA of 128 threads takes 128 rows (two M tiles per warp: a token tile's codes and records are loaded once for both)
// x 8 NT tokens and walks the groups in stages of eight through a two-stage cp.async ring.
#include "kernels.cuh"
#include <string.h>

namespace {

struct I4GMmaArgs {
    const uint8_t *w4; const float *scale;     // [O][I/2], [O][I/32]
    const int8_t *xi; const float *sx;         // row-quantized activations [S][I], [S]
    const int *rec;                            // [I/32][S8]: 0x4B400000 - 8 * sum of the codes of (group, token)
    float *y;                                  // [S][O]
    int S, S8, I, O;
};

constexpr int G_MAGIC = 0x4B400000;            // 1.5 * 2^23 as a float: see q4r4_mma.cu
constexpr float G_MAGIC_F = 12582912.0f;
constexpr int G_CH = 8;                        // groups per stage
// one stage: W [8 M tiles][16 rows] 144 bytes (8 groups x 16, padded: eight rows -> eight bank groups),
// D [8][16] 48 bytes (8 scales, padded likewise), B [tokens] 288 bytes (8 groups x 32, padded for 64-bit loads),
// R [tile][group][token pair] = {c0, c1, c0, c1}
constexpr int G_WROW = 144, G_W1 = 16 * G_WROW, G_DROW = 48, G_D1 = 16 * G_DROW, G_BTOK = 288, G_NSLOT = 8;
template <int NT> struct I4GStage {
    static constexpr int W = 0, D = G_NSLOT * G_W1, B = D + G_NSLOT * G_D1, R = B + NT * 8 * G_BTOK, BYTES = R + NT * G_CH * 64;
};

typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t g_pack2(float lo, float hi) { f32x2_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ f32x2_t g_pack2i(int lo, int hi) { f32x2_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r; }
__device__ __forceinline__ void g_unpack2(f32x2_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2_t g_add2(f32x2_t a, f32x2_t b) { f32x2_t r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2_t g_fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r;
}
__device__ __forceinline__ void g_mma_u8s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1,
                                           const int4 &ci) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(ci.x), "r"(ci.y), "r"(ci.z), "r"(ci.w));
}

template <int NT>
__global__ void __launch_bounds__(128) i4g_mma_kernel(I4GMmaArgs a) {
    using L = I4GStage<NT>;
    constexpr int MW = 2, NS = 2, NTHR = 128;
    extern __shared__ int4 smem_i4g[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(smem_i4g);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tid = lane & 3;
    const int I = a.I, nb = I / 32, O = a.O, S = a.S;
    const int n00 = blockIdx.y * NT * 8, row00 = blockIdx.x * 128;
    const int nstage = (nb + G_CH - 1) / G_CH;
    const int vw0 = warp * MW;
    // first group held by stage s: a partial last stage is shifted back so that it never runs past the row
    auto stage_g0 = [&](int s) { const int g0 = s * G_CH; return g0 + G_CH <= nb ? g0 : (nb >= G_CH ? nb - G_CH : 0); };
    auto fill_w = [&](int s) {                                 // codes: a warp instruction covers four rows x 128 contiguous bytes
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % NS) * L::BYTES;
        const int gs = stage_g0(s);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int r = i * 16 + (threadIdx.x >> 3), ch = threadIdx.x & 7;       // row of the CTA, group of the stage
            int row = row00 + r; row = row < O ? row : O - 1;
            if (nb >= G_CH || ch < nb)
                cp_async16(dst + L::W + (r >> 4) * G_W1 + (r & 15) * G_WROW + ch * 16, a.w4 + (size_t)row * (I / 2) + (size_t)(gs + ch) * 16);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {                          // scales: two per copy (the group count is even: 8-byte aligned)
            const int r = i * 32 + (threadIdx.x >> 2), pr = threadIdx.x & 3;
            int row = row00 + r; row = row < O ? row : O - 1;
            if (nb >= G_CH || pr * 2 < nb)
                cp_async8(dst + L::D + (r >> 4) * G_D1 + (r & 15) * G_DROW + pr * 8, a.scale + (size_t)row * nb + gs + pr * 2);
        }
    };
    auto fill_x = [&](int s) {                                 // activation side: codes and records of the CTA's tokens
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % NS) * L::BYTES;
        const int gs = stage_g0(s);
        for (int t = threadIdx.x; t < NT * 128; t += NTHR) {   // 16 chunks of 16 bytes per token
            const int tok = t >> 4, ch = t & 15;
            int n = n00 + tok; n = n < S ? n : S - 1;
            if (nb >= G_CH || ch * 16 < nb * 32)
                cp_async16(dst + L::B + tok * G_BTOK + ch * 16, a.xi + (size_t)n * I + (size_t)gs * 32 + ch * 16);
        }
        for (int t = threadIdx.x; t < NT * G_CH * 8; t += NTHR) {   // records: c of token k into both halves of its pair's entry
            const int j = t / (G_CH * 8), u = (t >> 3) % G_CH, k = t & 7;
            if (gs + u < nb && n00 + j * 8 + k < a.S8) {
                const int *src = a.rec + (size_t)(gs + u) * a.S8 + n00 + j * 8 + k;
                unsigned char *r = dst + L::R + j * G_CH * 64 + u * 64 + (k >> 1) * 16 + (k & 1) * 4;
                cp_async4(r, src);
                cp_async4(r + 8, src);
            }
        }
    };
    pdl_trigger();
    fill_w(0);                                                 // weights only: may overlap the previous kernel
    pdl_wait();                                                // codes and records come from the kernels before this one
    fill_x(0); cp_async_commit();

    f32x2_t acc[MW][NT][2];                                    // {(row_a, t0), (row_a, t1)} and {(row_b, t0), (row_b, t1)}
    const f32x2_t neg_magic = g_pack2(-G_MAGIC_F, -G_MAGIC_F);
#pragma unroll
    for (int m = 0; m < MW; m++)
#pragma unroll
        for (int j = 0; j < NT; j++) acc[m][j][0] = acc[m][j][1] = 0ull;
    const int offA = L::W + gid * G_WROW + tid * 4, offB = offA + 8 * G_WROW;
    const int offdA = L::D + gid * G_DROW, offdB = offdA + 8 * G_DROW;
    for (int s = 0; s < nstage; s++) {
        cp_async_wait<0>();                                    // this thread's copies of stage s have landed
        __syncthreads();                                       // everyone's have, and everyone is done with stage s - 1
        fill_w(s + 1); fill_x(s + 1); cp_async_commit();       // into the slot stage s - 1 used
        const unsigned char *st = smem + (size_t)(s % NS) * L::BYTES;
        const int g0 = s * G_CH, gs = stage_g0(s);
        auto group_step = [&](int ul) {                        // ul: position of the group inside the stage
            float sA[MW], sB[MW];
            unsigned a0[MW], a1[MW], a2[MW], a3[MW];
#pragma unroll
            for (int m = 0; m < MW; m++) {
                const unsigned char *sw = st + (vw0 + m) * G_W1, *sd = st + (vw0 + m) * G_D1;
                sA[m] = *reinterpret_cast<const float *>(sd + offdA + ul * 4);
                sB[m] = *reinterpret_cast<const float *>(sd + offdB + ul * 4);
                const unsigned wA = *reinterpret_cast<const unsigned *>(sw + offA + ul * 16);
                const unsigned wB = *reinterpret_cast<const unsigned *>(sw + offB + ul * 16);
                a0[m] = wA & 0x0f0f0f0fu; a2[m] = (wA >> 4) & 0x0f0f0f0fu;      // even elements, odd elements
                a1[m] = wB & 0x0f0f0f0fu; a3[m] = (wB >> 4) & 0x0f0f0f0fu;
            }
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const uint2 xv = *reinterpret_cast<const uint2 *>(st + L::B + (j * 8 + gid) * G_BTOK + ul * 32 + tid * 8);
                const unsigned b0 = __byte_perm(xv.x, xv.y, 0x6420), b1 = __byte_perm(xv.x, xv.y, 0x7531);
                const int4 ci = *reinterpret_cast<const int4 *>(st + L::R + j * G_CH * 64 + ul * 64 + tid * 16);   // {c0, c1, c0, c1} of tokens t0, t1
#pragma unroll
                for (int m = 0; m < MW; m++) {
                    int c[4];
                    g_mma_u8s8(c, a0[m], a1[m], a2[m], a3[m], b0, b1, ci);
                    const f32x2_t fa = g_add2(g_pack2i(c[0], c[1]), neg_magic), fb = g_add2(g_pack2i(c[2], c[3]), neg_magic);
                    acc[m][j][0] = g_fma2(g_pack2(sA[m], sA[m]), fa, acc[m][j][0]);   // hw/hw_quant.h:47: acc += scl[g] * (float)d
                    acc[m][j][1] = g_fma2(g_pack2(sB[m], sB[m]), fb, acc[m][j][1]);
                }
            }
        };
        if (g0 + G_CH <= nb) {
#pragma unroll
            for (int u = 0; u < G_CH; u++) group_step(u);
        } else {
            for (int g = g0; g < nb; g++) group_step(g - gs);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int m = 0; m < MW; m++) {
        const int row_a = row00 + (vw0 + m) * 16 + gid, row_b = row_a + 8;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const int t0 = n00 + j * 8 + tid * 2, t1 = t0 + 1;
            float ya0, ya1, yb0, yb1;
            g_unpack2(acc[m][j][0], ya0, ya1);
            g_unpack2(acc[m][j][1], yb0, yb1);
            if (t0 < S) {                                      // nn/matmul.c:157: sx * dot
                const float sx = a.sx[t0];
                if (row_a < O) a.y[(size_t)t0 * O + row_a] = __fmul_rn(sx, ya0);
                if (row_b < O) a.y[(size_t)t0 * O + row_b] = __fmul_rn(sx, yb0);
            }
            if (t1 < S) {
                const float sx = a.sx[t1];
                if (row_a < O) a.y[(size_t)t1 * O + row_a] = __fmul_rn(sx, ya1);
                if (row_b < O) a.y[(size_t)t1 * O + row_b] = __fmul_rn(sx, yb1);
            }
        }
    }
}

// records [group][token] (token count padded to 8, padding zeroed)
__global__ void __launch_bounds__(256) i4g_rec_kernel(const int8_t *__restrict__ xi, int *__restrict__ rec, int S, int S8, int I) {
    pdl_wait();                                   // (no early trigger: the product after this one is not persistent)
    const int nb = I / 32;
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)S8 * nb) return;
    const int g = (int)(i / S8), t = (int)(i - (long long)g * S8);
    int r = 0;
    if (t < S) {
        const int4 *p = reinterpret_cast<const int4 *>(xi + (size_t)t * I + (size_t)g * 32);
        const int4 u = p[0], v = p[1];
        int sum = __dp4a(u.x, 0x01010101, 0);
        sum = __dp4a(u.y, 0x01010101, sum); sum = __dp4a(u.z, 0x01010101, sum); sum = __dp4a(u.w, 0x01010101, sum);
        sum = __dp4a(v.x, 0x01010101, sum); sum = __dp4a(v.y, 0x01010101, sum);
        sum = __dp4a(v.z, 0x01010101, sum); sum = __dp4a(v.w, 0x01010101, sum);
        r = G_MAGIC - 8 * sum;
    }
    rec[i] = r;
}

template <int NT>
int launch_i4g_mma_t(const I4GMmaArgs &a, cudaStream_t st) {
    constexpr int SMEM = 2 * I4GStage<NT>::BYTES;
    static bool attr_done[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "i4g_mma: device %d", dev);
    if (!attr_done[dev]) {
        CK(cudaFuncSetAttribute(i4g_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_done[dev] = true;
    }
    dim3 grid((a.O + 127) / 128, (a.S + 8 * NT - 1) / (8 * NT));
    if (grid.y > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "i4g_mma: S=%d in one call", a.S);
    CK(moty_launch_pdl(i4g_mma_kernel<NT>, grid, dim3(128), (size_t)SMEM, st, a));
    return 0;
}

}  // namespace

size_t i4g_mma_scratch_bytes(int S, int I) { return (size_t)((S + 7) / 8 * 8) * (I / 32) * 4; }

// xi/sx: the S rows quantized per row (qrow_i8); rec: scratch of i4g_mma_scratch_bytes(S, I).
// I a multiple of 64 (even group count, 16-byte aligned code rows), I <= MOTY_QROW_MAX.
int launch_i4g_mma(const uint8_t *w4, const float *scale, const int8_t *xi, const float *sx, int *rec, float *y,
                   int S, int I, int O, int sms, cudaStream_t st) {
    if (I % 64 != 0 || I <= 0 || I > MOTY_QROW_MAX || S <= 0 || O <= 0)
        return moty_set_error(MOTY_CUDA_EARG, "i4g_mma: S=%d I=%d O=%d", S, I, O);
    const int nb = I / 32, S8 = (S + 7) / 8 * 8;
    const long long nrec = (long long)S8 * nb;
    CK(moty_launch_pdl(i4g_rec_kernel, dim3((unsigned)((nrec + 255) / 256)), dim3(256), (size_t)0, st, xi, rec, S, S8, I));
    I4GMmaArgs a;
    a.w4 = w4; a.scale = scale; a.xi = xi; a.sx = sx; a.rec = rec; a.y = y; a.S = S; a.S8 = S8; a.I = I; a.O = O;
    // more N tiles per CTA amortise the weight traffic and unpack; fewer give more CTAs (never a tile wider than the batch)
    const long long mct = (O + 127) / 128, want = (long long)sms * 2;
    const bool nt4 = S > 16 && mct * ((S + 31) / 32) >= want, nt2 = S > 8 && mct * ((S + 15) / 16) >= want;
    if (nt4) return launch_i4g_mma_t<4>(a, st);
    if (nt2) return launch_i4g_mma_t<2>(a, st);
    return launch_i4g_mma_t<1>(a, st);
}
