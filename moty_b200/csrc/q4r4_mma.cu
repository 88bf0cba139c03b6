// q4r4_mma.cu -- Q4R4 weights x a batch of group-quantized activation rows (S >= 5).
//
// Replaces moty_matmul_q4r4_s (nn/matmul.c:405-433) with its two kernels
// moty_hw_q4r4_gemm_ref / _gemm4t_ref (hw/hw_q4r4.h:47-84) for batches.
//
// The arithmetic has two layers.  Inside one group of 32 weights the reference sums
// integers: exact in any order.  Across groups it adds ONE f32 term per group to a
// running sum, in ascending group order: that chain has to be reproduced step by step.
// So the integer layer goes to the tensor cores one group at a time -- a K = 32 integer
// MMA is exactly one group -- and its int32 result is consumed in registers by the f32
// chain before the next group: mma.sync.m16n8k32 (u8 nibble codes x s8 activation codes ->
// s32), 16 weight rows x 8 tokens per instruction, accumulator fragments in registers.
// (tcgen05 keeps accumulators in TMEM; reading a whole tile back after every K = 32 step
// costs more than the MMA saves, and the chain, three or four f32 operations per output and
// group, is the bound either way.)
//
// Fragment fit: the 16 rows of an M tile are four Q4R4 blocks.  A block stores, per row and
// group, 16 bytes with byte j = code[j] | code[j+16] << 4; the A fragment wants from thread
// (gid, tid) the codes k = 4 tid .. 4 tid + 3 (a0/a1) and k = 16 + 4 tid .. (a2/a3) of rows
// gid and gid + 8: that is ONE 32-bit word per row, low nibbles -> a0/a1, high -> a2/a3.
// Weights, activation codes and the chain records all reach the warps through a ring of
// shared-memory stages filled by cp.async (eight groups per stage), so no load sits in the chain.
//
// The reference has two formulas for a group's term; which one a token gets depends on its place
// in its 32-token tile (nn/matmul.c:424-432):
//   token-by-token (hw/hw_q4r4.h:58-59):  acc = fma((float)(sum - 8*xsum), d*xs, acc)
//   4-token tile   (hw/hw_q4r4.h:78-81):  acc = fma((float)sum, d*xs, acc); acc = fma(-d, (8*xsum)*xs, acc)
// Per (group, token) a 16-byte record {xs, c, nv, -} prepared by q4r4_rec_kernel carries both without a branch:
//   c  = 0x4B400000 - 8*xsum (token-by-token) or 0x4B400000 (tile): the MMA's accumulator INPUT, so the instruction
//        returns the bit pattern of the float 1.5 * 2^23 + (sum - 8*xsum) or 1.5 * 2^23 + sum, and one exact FADD of
//        -1.5 * 2^23 leaves (float)(sum - 8*xsum) or (float)sum: no integer add, no conversion unit;
//   nv = -((8*xsum)*xs) (tile) or +0 (token-by-token): the second step is acc = fma(d, nv, acc) for every token --
//        fma(d, -v, acc) is fma(-d, v, acc) bit for bit, and adding d * 0 leaves acc as it is.
// The steps -- FADD, FMUL (d*xs), FFMA, FFMA -- run as packed add/mul/fma.rn.f32x2 instructions, two tokens each: every
// lane rounds like the scalar instruction, so the bits are the reference's at half the issue slots.
//
// RELAX (opt-in, moty_cuda_set_q4r4_batch_relaxed): every token takes the token-by-token formula, and the second FFMA
// and the nv half of the record are gone.  Tokens the reference treats that way keep their bits; the others move by
// the rounding of one FFMA per group.  Q8R4 has no offset term: one formula, RELAX or not.
#include "kernels.cuh"
#include <string.h>

struct Q4MmaArgs {
    const uint8_t *w; const uint16_t *d;
    const int8_t *xq;                         // codes [S][I]
    const int *rec;                           // records [I/32][S8] of 4 ints {xs, c, nv, -}, or of 2 ints {xs, c} when there is one formula; S8 = S rounded up to 8
    float *y; int ldy;
    int S, S8, I, O;
    // grouped mode (MoE batches): CTA row y of the grid is a tile = up to 8 NT consecutive rows of the
    // gathered batch that share one expert's matrix; xq rows are found through xmap (null: identity)
    const Q4Tile *tiles; const int *ntiles_dev; const int *xmap;
};

// D = A (16x32 u8 or s8, row) * B (32x8 s8, col) + C, C = the four registers of one 128-bit load:
// {c0, c1} for rows gid and gid + 8 alike
__device__ __forceinline__ void mma_u8s8_16832_c4(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                                  unsigned b0, unsigned b1, const int4 &ci) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(ci.x), "r"(ci.y), "r"(ci.z), "r"(ci.w));
}
__device__ __forceinline__ void mma_s8s8_16832_c4(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                                  unsigned b0, unsigned b1, const int4 &ci) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(ci.x), "r"(ci.y), "r"(ci.z), "r"(ci.w));
}

// int -> float for |i| < 2^22 without the conversion unit (a quarter-rate pipe that the chain would saturate):
// 0x4B400000 is 1.5 * 2^23 as a float; adding i to its bit pattern gives the float 1.5 * 2^23 + i exactly, and the
// subtraction is exact.  Group sums are below 2^17 in magnitude.
constexpr int Q4_MAGIC = 0x4B400000;
constexpr float Q4_MAGIC_F = 12582912.0f;

// two f32 lanes per instruction
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack2(float lo, float hi) {
    f32x2_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi)); return r;
}
__device__ __forceinline__ f32x2_t pack2i(int lo, int hi) {
    f32x2_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r;
}
__device__ __forceinline__ void unpack2(f32x2_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2_t add2(f32x2_t a, f32x2_t b) { f32x2_t r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2_t mul2(f32x2_t a, f32x2_t b) { f32x2_t r; asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ f32x2_t fma2(f32x2_t a, f32x2_t b, f32x2_t c) {
    f32x2_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r;
}

// A CTA takes NSLOT M tiles (16 weight rows each; MW per warp) x NT N tiles (8 NT tokens) and walks the groups in
// stages of GCH = 8.  One stage in shared memory:
//   W  per M tile: its four blocks' codes, 4 x 512 bytes, each block padded by 64 bytes so that the two
//      blocks a fragment load touches sit in different banks
//   D  per M tile: 4 x 64 bytes of f16 scales
//   B  the tokens' codes, 256 bytes per token, token stride 272 bytes (eight tokens -> eight bank groups)
//   R  [tile][group][token pair] = {c0, c1, c0, c1}: the MMA's accumulator input as ONE 128-bit load
//   RX [tile][group][token pair] = {xs0, xs1, nv0, nv1}, or {xs0, xs1} when there is one formula
constexpr int GCH = 8;
constexpr int STG_D1 = 4 * 64, BTOK = 272;
// Q8 = the int8 sibling Q8R4 (hw/hw_q4r4.h:92-130): 128 bytes per (block, group) = 4 rows x 32 signed codes, no
// offset term, the same chain.  Its blocks are padded by 16 bytes: a row's fragment words sit 32 bytes apart,
// so the second block of a fragment load has to land 16 bytes off to miss the banks of the first.
template <int NT, bool Q8, int NSLOT, bool TWO> struct Q4Stage {
    static constexpr int GB = Q8 ? 128 : 64;                   // bytes per (block, group)
    static constexpr int WBLK = Q8 ? GCH * 128 + 16 : GCH * 64 + 64, STG_W1 = 4 * WBLK;
    static constexpr int RXB = TWO ? 16 : 8;                   // bytes per token pair in RX
    static constexpr int W = 0, D = NSLOT * STG_W1, B = D + NSLOT * STG_D1, R = B + NT * 8 * BTOK, RX = R + NT * GCH * 64;
    static constexpr int BYTES = RX + NT * GCH * 4 * RXB;
};

// MW = M tiles per warp, NW = warps per CTA, NS = ring stages.  With two M tiles a warp loads a token tile's codes and
// records once for both: the 128-bit record loads are four shared-memory wavefronts each however few bytes they move
// (four lanes share them), and at one M tile per warp they, not the issue slots, set the pace.
template <int NT, bool Q8, bool RELAX, int MW, int NS, int NW>
__global__ void __launch_bounds__(32 * NW) q4r4_mma_kernel(Q4MmaArgs a) {
    constexpr bool TWO = !RELAX && !Q8;                        // both formulas: the second FFMA and the nv half of RX
    constexpr int NSLOT = NW * MW, NTHR = 32 * NW;
    using L = Q4Stage<NT, Q8, NSLOT, TWO>;
    constexpr int GB = L::GB, WBLK = L::WBLK, STG_W1 = L::STG_W1;
    extern __shared__ int4 smem_q4mma[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(smem_q4mma);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tid = lane & 3;
    const int I = a.I, nb = I / 32, O = a.O;
    const uint8_t *Wp = a.w; const uint16_t *Dp = a.d;
    int n00 = blockIdx.y * NT * 8, S = a.S;                    // first token of the CTA, end of its token range
    pdl_trigger();
    if (a.tiles) {
        pdl_wait();                                            // the tile table comes from the plan kernel
        if ((int)blockIdx.y >= *a.ntiles_dev) return;          // CTA-uniform
        const Q4Tile t = a.tiles[blockIdx.y];
        Wp = t.w; Dp = t.d; n00 = t.row0; S = t.row0 + t.nrows;
    }
    const int nblk = (O + 3) / 4, nstage = (nb + GCH - 1) / GCH;
    // the warp's M tiles are slots vw0 .. vw0 + MW - 1 of the CTA's (a tile may lie past the end: it is still copied)
    const int vw0 = warp * MW, mt0 = blockIdx.x * NSLOT + vw0;
    // where this thread's fragment words and scales sit inside a stage, for M-tile slot 0
    const int ba_l = gid >> 2, bb_l = ba_l + 2, rr = gid & 3;
    const int offA = L::W + ba_l * WBLK + rr * (GB / 4) + tid * 4, offB = L::W + bb_l * WBLK + rr * (GB / 4) + tid * 4;
    const int offdA = L::D + ba_l * 64 + rr * 2, offdB = L::D + bb_l * 64 + rr * 2;
    // first group held by stage s: a partial last stage is shifted back so that it never runs past the row
    auto stage_g0 = [&](int s) { const int g0 = s * GCH; return g0 + GCH <= nb ? g0 : (nb >= GCH ? nb - GCH : 0); };
    auto fill_w = [&](int s) {                                 // weights: lane l copies int4 number l of each block, and 8 bytes of scales
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % NS) * L::BYTES;
        const int gs = stage_g0(s);
#pragma unroll
        for (int m = 0; m < MW; m++) {
            const int vw = vw0 + m, mt = mt0 + m;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                int blk = mt * 4 + q; blk = blk < nblk ? blk : nblk - 1;
#pragma unroll
                for (int h = 0; h < GB / 64; h++) {            // 512 bytes per round of the warp
                    const int off = h * 512 + lane * 16;
                    if (nb >= GCH || off < nb * GB)
                        cp_async16(dst + L::W + vw * STG_W1 + q * WBLK + off, Wp + ((size_t)blk * nb + gs) * GB + off);
                }
            }
            const int q = lane >> 3, part = lane & 7;
            int blk = mt * 4 + q; blk = blk < nblk ? blk : nblk - 1;
            if (nb >= GCH || part < nb)
                cp_async8(dst + L::D + vw * STG_D1 + q * 64 + part * 8, Dp + ((size_t)blk * nb + gs) * 4 + part * 4);
        }
    };
    auto fill_x = [&](int s) {                                 // activation side: codes and records of the CTA's tokens
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % NS) * L::BYTES;
        const int gs = stage_g0(s);
        for (int t = threadIdx.x; t < NT * 128; t += NTHR) {   // 16 chunks of 16 bytes per token
            const int tok = t >> 4, ch = t & 15;
            int n = n00 + tok; n = n < S ? n : S - 1;
            if (a.xmap) n = a.xmap[n];
            if (nb >= GCH || ch * 16 < nb * 32)
                cp_async16(dst + L::B + tok * BTOK + ch * 16, a.xq + (size_t)n * I + (size_t)gs * 32 + ch * 16);
        }
        // record {xs, c[, nv, -]} of token k (a tile of the grouped mode may start at an odd row, so token by token):
        // c into both halves of its pair's R entry, xs and nv into the pair's RX entry.  Tokens past the batch (or the
        // tile): nothing copied, nothing stored at the end.
        // (Two loops and plain sums of offsets, here and in the loads below, on purpose: with one loop over a record size,
        // or the offsets written as (j * GCH + u) * 64, the compiler's schedule of the main loop came out 6 % slower on
        // the one-formula kernels -- 240 against 225 us on 15360 x 3840 at S = 512, same instructions.)
        if (!TWO) {
            for (int t = threadIdx.x; t < NT * GCH * 8; t += NTHR) {
                const int j = t / (GCH * 8), u = (t >> 3) % GCH, k = t & 7;
                if (gs + u < nb && n00 + j * 8 + k < (a.tiles ? S : a.S8)) {
                    const int *src = reinterpret_cast<const int *>(reinterpret_cast<const int2 *>(a.rec) + (size_t)(gs + u) * a.S8 + n00 + j * 8 + k);
                    unsigned char *r = dst + L::R + j * GCH * 64 + u * 64 + (k >> 1) * 16 + (k & 1) * 4;
                    cp_async4(dst + L::RX + j * GCH * 32 + u * 32 + k * 4, src);
                    cp_async4(r, src + 1);
                    cp_async4(r + 8, src + 1);
                }
            }
        } else {
            for (int t = threadIdx.x; t < NT * GCH * 8; t += NTHR) {
                const int j = t / (GCH * 8), u = (t >> 3) % GCH, k = t & 7;
                if (gs + u < nb && n00 + j * 8 + k < (a.tiles ? S : a.S8)) {
                    const int *src = reinterpret_cast<const int *>(reinterpret_cast<const int4 *>(a.rec) + (size_t)(gs + u) * a.S8 + n00 + j * 8 + k);
                    unsigned char *r = dst + L::R + j * GCH * 64 + u * 64 + (k >> 1) * 16 + (k & 1) * 4;
                    unsigned char *x = dst + L::RX + j * GCH * 64 + u * 64 + (k >> 1) * 16 + (k & 1) * 4;
                    cp_async4(x, src);
                    cp_async4(r, src + 1);
                    cp_async4(r + 8, src + 1);
                    cp_async4(x + 8, src + 2);
                }
            }
        }
    };
#pragma unroll
    for (int i = 0; i < NS - 1; i++) fill_w(i);                // weights only: may overlap the previous kernel
    pdl_wait();                                                // codes and records come from the kernels before this one
#pragma unroll
    for (int i = 0; i < NS - 1; i++) { fill_x(i); cp_async_commit(); }

    f32x2_t acc[MW][NT][2];                                    // {(row_a, t0), (row_a, t1)} and {(row_b, t0), (row_b, t1)}
    const f32x2_t neg_magic = pack2(-Q4_MAGIC_F, -Q4_MAGIC_F);
#pragma unroll
    for (int m = 0; m < MW; m++)
#pragma unroll
        for (int j = 0; j < NT; j++) acc[m][j][0] = acc[m][j][1] = 0ull;
    for (int s = 0; s < nstage; s++) {
        cp_async_wait<NS - 2>();                               // this thread's copies of stage s have landed
        __syncthreads();                                       // everyone's have, and everyone is done with stage s - 1
        fill_w(s + NS - 1); fill_x(s + NS - 1); cp_async_commit();   // into the slot stage s - 1 used
        const unsigned char *st = smem + (size_t)(s % NS) * L::BYTES;
        const int g0 = s * GCH, gs = stage_g0(s);
        auto group_step = [&](int ul) {                        // ul: position of the group inside the stage
            float dA[MW], dB[MW];
            unsigned a0[MW], a1[MW], a2[MW], a3[MW];
#pragma unroll
            for (int m = 0; m < MW; m++) {
                const unsigned char *sw = st + (vw0 + m) * STG_W1, *sd = st + (vw0 + m) * STG_D1;
                dA[m] = f16bits_to_f32(*reinterpret_cast<const uint16_t *>(sd + offdA + ul * 8));
                dB[m] = f16bits_to_f32(*reinterpret_cast<const uint16_t *>(sd + offdB + ul * 8));
                if (Q8) {                                      // a row's codes k = 4 tid .. and k = 16 + 4 tid ..: two words
                    a0[m] = *reinterpret_cast<const unsigned *>(sw + offA + ul * GB); a2[m] = *reinterpret_cast<const unsigned *>(sw + offA + ul * GB + 16);
                    a1[m] = *reinterpret_cast<const unsigned *>(sw + offB + ul * GB); a3[m] = *reinterpret_cast<const unsigned *>(sw + offB + ul * GB + 16);
                } else {                                       // one word: low nibbles -> a0/a1, high nibbles -> a2/a3
                    const unsigned wA = *reinterpret_cast<const unsigned *>(sw + offA + ul * GB);
                    const unsigned wB = *reinterpret_cast<const unsigned *>(sw + offB + ul * GB);
                    a0[m] = wA & 0x0f0f0f0fu; a2[m] = (wA >> 4) & 0x0f0f0f0fu;
                    a1[m] = wB & 0x0f0f0f0fu; a3[m] = (wB >> 4) & 0x0f0f0f0fu;
                }
            }
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const unsigned char *bp = st + L::B + (j * 8 + gid) * BTOK + ul * 32 + tid * 4;
                const unsigned b0 = *reinterpret_cast<const unsigned *>(bp), b1 = *reinterpret_cast<const unsigned *>(bp + 16);
                const int4 ci = *reinterpret_cast<const int4 *>(st + L::R + j * GCH * 64 + ul * 64 + tid * 16);   // {c0, c1, c0, c1} of tokens t0, t1
                f32x2_t xs2 = 0ull, nv2 = 0ull;
                if (!TWO) xs2 = *reinterpret_cast<const f32x2_t *>(st + L::RX + j * GCH * 32 + ul * 32 + tid * 8);
                if (TWO) {
                    const int4 e = *reinterpret_cast<const int4 *>(st + L::RX + j * GCH * 64 + ul * 64 + tid * 16);
                    xs2 = pack2i(e.x, e.y); nv2 = pack2i(e.z, e.w);
                }
#pragma unroll
                for (int m = 0; m < MW; m++) {
                    int c[4];
                    if (Q8) mma_s8s8_16832_c4(c, a0[m], a1[m], a2[m], a3[m], b0, b1, ci);
                    else mma_u8s8_16832_c4(c, a0[m], a1[m], a2[m], a3[m], b0, b1, ci);
                    const f32x2_t fa = add2(pack2i(c[0], c[1]), neg_magic), fb = add2(pack2i(c[2], c[3]), neg_magic);
                    const f32x2_t da2 = pack2(dA[m], dA[m]), db2 = pack2(dB[m], dB[m]);
                    acc[m][j][0] = fma2(fa, mul2(da2, xs2), acc[m][j][0]);
                    acc[m][j][1] = fma2(fb, mul2(db2, xs2), acc[m][j][1]);
                    if (TWO) {
                        acc[m][j][0] = fma2(da2, nv2, acc[m][j][0]);
                        acc[m][j][1] = fma2(db2, nv2, acc[m][j][1]);
                    }
                }
            }
        };
        if (g0 + GCH <= nb) {
#pragma unroll
            for (int u = 0; u < GCH; u++) group_step(u);
        } else {
            for (int g = g0; g < nb; g++) group_step(g - gs);
        }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int m = 0; m < MW; m++) {
        const int row_a = (mt0 + m) * 16 + gid, row_b = row_a + 8;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const int t0 = n00 + j * 8 + tid * 2, t1 = t0 + 1;
            float ya0, ya1, yb0, yb1;
            unpack2(acc[m][j][0], ya0, ya1);
            unpack2(acc[m][j][1], yb0, yb1);
            if (t0 < S) {
                if (row_a < O) a.y[(size_t)t0 * a.ldy + row_a] = ya0;
                if (row_b < O) a.y[(size_t)t0 * a.ldy + row_b] = yb0;
            }
            if (t1 < S) {
                if (row_a < O) a.y[(size_t)t1 * a.ldy + row_a] = ya1;
                if (row_b < O) a.y[(size_t)t1 * a.ldy + row_b] = yb1;
            }
        }
    }
}

// one record: tile = the token takes the 4-token-tile formula
__device__ __forceinline__ int4 q4_record(float sc, int sm, bool tile) {
    int4 r;
    r.x = __float_as_int(sc);
    r.y = tile ? Q4_MAGIC : Q4_MAGIC - 8 * sm;
    r.z = tile ? __float_as_int(-__fmul_rn(__fmul_rn(8.f, (float)sm), sc)) : 0;
    r.w = 0;
    return r;
}

// records of the chain step, [group][token] (token count padded to 8, padding zeroed).  Which formula:
// moty_matmul_q4r4_s cuts the batch into tiles of 32 tokens and sends the first (size / 4 * 4) tokens of a tile
// through the 4-token kernel, the rest through the token-by-token kernel (nn/matmul.c:424-432); relax: all through the latter
__global__ void __launch_bounds__(256) q4r4_rec_kernel(const float *__restrict__ xs, const int32_t *__restrict__ xsum,
                                                       int *__restrict__ rec, int S, int S8, int nb, int q8, int relax) {
    pdl_wait();                                   // (no early trigger: the product after this one is not persistent, and its
                                                  // CTAs spread unevenly when they arrive while others are still resident)
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)S8 * nb) return;
    const int g = (int)(i / S8), t = (int)(i - (long long)g * S8);
    int4 r = make_int4(0, 0, 0, 0);
    if (t < S) {
        const int t0 = t / 32 * 32;
        const int ns = S - t0 < 32 ? S - t0 : 32;
        const bool tile = !q8 && !relax && (t - t0) < ns / 4 * 4;        // Q8R4 has one formula and no offset term
        r = q4_record(xs[(size_t)t * nb + g], q8 ? 0 : xsum[(size_t)t * nb + g], tile);
    }
    if (q8 || relax) reinterpret_cast<int2 *>(rec)[i] = make_int2(r.x, r.y);    // one formula: the short record
    else reinterpret_cast<int4 *>(rec)[i] = r;
}

template <int NT, bool Q8, bool RELAX, int MW, int NS, int NW>
static int launch_mma_tm(const Q4MmaArgs &a, cudaStream_t st, int ntiles_max) {
    constexpr int NSLOT = NW * MW, SMEM = NS * Q4Stage<NT, Q8, NSLOT, !RELAX && !Q8>::BYTES;
    static bool attr_done[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q4r4_mma: device %d", dev);
    if (!attr_done[dev]) {
        CK(cudaFuncSetAttribute(q4r4_mma_kernel<NT, Q8, RELAX, MW, NS, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_done[dev] = true;
    }
    const int nmt = (a.O + 15) / 16;
    dim3 grid((nmt + NSLOT - 1) / NSLOT, a.tiles ? ntiles_max : (a.S + 8 * NT - 1) / (8 * NT));
    if (grid.y > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "q4r4_mma: S=%d in one call", a.S);
    CK(moty_launch_pdl(q4r4_mma_kernel<NT, Q8, RELAX, MW, NS, NW>, grid, dim3(32 * NW), (size_t)SMEM, st, a));
    return 0;
}
// Two M tiles per warp and two stages of about 32 KB (three CTAs of 128 threads per SM: the kernel is bound by latency,
// not by bytes); 128 rows per CTA, or 256 when 128-row CTAs would come to between one and three resident sets of 3 per
// SM (measured: 3840 x 15360 at S = 512 285 vs 320 us; no difference on larger grids).
template <int NT, bool Q8, bool RELAX>
static int launch_mma_t(const Q4MmaArgs &a, cudaStream_t st, int sms, int ntiles_max = 0) {
    const long long rows = a.tiles ? ntiles_max : (a.S + 8 * NT - 1) / (8 * NT);
    const long long ctas4 = ((a.O + 15) / 16 + 7) / 8 * rows, slots = 3LL * sms;
    // fewer CTAs than SMs (a few tokens x a matrix of few, long rows): the call streams the weights through a handful of
    // CTAs, and what counts is bytes in flight per CTA: eight warps, one M tile each, three stages
    // (3840 x 15360 at S = 16: 60 CTAs, 60 us against 71)
    if (ctas4 < sms) return launch_mma_tm<NT, Q8, RELAX, 1, 3, 8>(a, st, ntiles_max);
    if (ctas4 > slots && ctas4 < 3 * slots) return launch_mma_tm<NT, Q8, RELAX, 2, 2, 8>(a, st, ntiles_max);
    return launch_mma_tm<NT, Q8, RELAX, 2, 2, 4>(a, st, ntiles_max);
}
// Q8R4 has one formula: the relaxed instantiation serves it either way
template <int NT>
static int launch_mma_nt(const Q4MmaArgs &a, cudaStream_t st, int sms, int q8, int relax, int ntiles_max = 0) {
    if (q8) return launch_mma_t<NT, true, true>(a, st, sms, ntiles_max);
    if (relax) return launch_mma_t<NT, false, true>(a, st, sms, ntiles_max);
    return launch_mma_t<NT, false, false>(a, st, sms, ntiles_max);
}

// xq/xs/xsum: the group-quantized batch; rec: scratch for (I/32) * ceil8(S) records of 16 bytes (8 are used when there is one formula)
// q8 != 0: w holds Q8R4 codes (128 bytes per block and group)
// relax != 0: the token-by-token formula for every token (see the head of this file)
int launch_q4r4_mma(const uint8_t *w, const uint16_t *d, const int8_t *xq, const float *xs, const int32_t *xsum,
                    int4 *rec, float *y, int ldy, int S, int I, int O, int q8, int sms, cudaStream_t st, int relax) {
    if (I % 32 != 0 || I <= 0 || S <= 0) return moty_set_error(MOTY_CUDA_EARG, "q4r4_mma: S=%d I=%d", S, I);
    if (O <= 0) return 0;
    const int nb = I / 32, S8 = (S + 7) / 8 * 8;
    const long long nrec = (long long)S8 * nb;
    CK(moty_launch_pdl(q4r4_rec_kernel, dim3((unsigned)((nrec + 255) / 256)), dim3(256), (size_t)0, st, xs, xsum, reinterpret_cast<int *>(rec), S, S8, nb, q8, relax));
    Q4MmaArgs a; memset(&a, 0, sizeof a);
    a.w = w; a.d = d; a.xq = xq; a.rec = reinterpret_cast<const int *>(rec); a.y = y; a.ldy = ldy; a.S = S; a.S8 = S8; a.I = I; a.O = O;
    // more N tiles per CTA amortise the weight traffic and unpack; fewer give more CTAs: keep ~2 CTAs per SM
    const long long mct = ((O + 15) / 16 + 7) / 8, want = (long long)sms * 2;
    // (never a tile wider than the batch: its empty token columns would cost the same chain work)
    const bool nt4 = S > 16 && mct * ((S + 31) / 32) >= want, nt2 = S > 8 && mct * ((S + 15) / 16) >= want;
    if (nt4) return launch_mma_nt<4>(a, st, sms, q8, relax);
    if (nt2) return launch_mma_nt<2>(a, st, sms, q8, relax);
    return launch_mma_nt<1>(a, st, sms, q8, relax);
}

// records of a gathered batch: row p of the batch is row xmap[p] (null: p) of xs/xsum, its formula
// flag form[p] comes with the plan; rows at and past *npairs_dev are zero
__global__ void __launch_bounds__(256) q4r4_rec_gather_kernel(const float *__restrict__ xs, const int32_t *__restrict__ xsum,
                                                              const int *__restrict__ xmap, const uint8_t *__restrict__ form,
                                                              const int *__restrict__ npairs_dev, int *__restrict__ rec,
                                                              int P8, int nb, int relax) {
    pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= (long long)P8 * nb) return;
    const int g = (int)(i / P8), p = (int)(i - (long long)g * P8);
    int4 r = make_int4(0, 0, 0, 0);
    if (p < *npairs_dev) {
        const int t = xmap ? xmap[p] : p;
        r = q4_record(xs[(size_t)t * nb + g], xsum[(size_t)t * nb + g], !relax && form[p] != 0);
    }
    if (relax) reinterpret_cast<int2 *>(rec)[i] = make_int2(r.x, r.y);
    else reinterpret_cast<int4 *>(rec)[i] = r;
}

// Grouped products of a MoE batch: tiles[i] = {expert matrix, first row, rows <= tile_rows} over a
// gathered batch of at most P rows (tile_rows is 8, 16 or 32 and is what the plan was built with).
// y row p receives the product for batch row p.  xs/xsum are indexed like xq (through xmap).
int launch_q4r4_mma_grouped(const Q4Tile *tiles, const int *ntiles_dev, int ntiles_max, int tile_rows,
                            const int *npairs_dev, const int8_t *xq, const float *xs, const int32_t *xsum,
                            const int *xmap, const uint8_t *form, int4 *rec, int build_rec, float *y, int ldy, int P,
                            int I, int O, cudaStream_t st, int relax, int sms) {
    if (I % 32 != 0 || I <= 0 || P <= 0 || (tile_rows != 8 && tile_rows != 16 && tile_rows != 32))
        return moty_set_error(MOTY_CUDA_EARG, "q4r4_mma_grouped: P=%d I=%d tile=%d", P, I, tile_rows);
    if (O <= 0 || ntiles_max <= 0) return 0;
    if (ntiles_max > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "q4r4_mma_grouped: %d tiles in one call", ntiles_max);
    const int nb = I / 32, P8 = (P + 7) / 8 * 8;
    const long long nrec = (long long)P8 * nb;
    if (build_rec) {                                           // gate and up share the records of the gathered input
        CK(moty_launch_pdl(q4r4_rec_gather_kernel, dim3((unsigned)((nrec + 255) / 256)), dim3(256), (size_t)0, st, xs, xsum, xmap, form,
                           npairs_dev, reinterpret_cast<int *>(rec), P8, nb, relax));
    }
    Q4MmaArgs a; memset(&a, 0, sizeof a);
    a.xq = xq; a.rec = reinterpret_cast<const int *>(rec); a.y = y; a.ldy = ldy; a.S = P; a.S8 = P8; a.I = I; a.O = O;
    a.tiles = tiles; a.ntiles_dev = ntiles_dev; a.xmap = xmap;
    if (tile_rows == 32) return launch_mma_nt<4>(a, st, sms, 0, relax, ntiles_max);
    if (tile_rows == 16) return launch_mma_nt<2>(a, st, sms, 0, relax, ntiles_max);
    return launch_mma_nt<1>(a, st, sms, 0, relax, ntiles_max);
}
