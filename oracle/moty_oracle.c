/* moty_oracle.c -- CPU restatement of moty's quantized-matmul hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against; it is never linked into, imported by or called from the
 * shipped library.  Only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may load it.
 *
 * Every function restates, in plain scalar C, what the named reference
 * function computes (file:line refer to the moty source tree, directory c/).
 * The restatement is pinned two ways: against the committed golden vectors
 * (tests/golden, produced by the reference's own compiled code) and, where the
 * reference build is present, bit-for-bit against that build.
 *
 * Floating-point contract: the reference is built by gcc in GNU mode for a
 * machine with FMA, so `acc += a * b` in its sources is one fused
 * multiply-add.  This file is compiled with -ffp-contract=off and spells every
 * such step as fmaf(), so its results do not depend on compiler flags.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* f16 <-> f32                                                          */
/* ------------------------------------------------------------------ */

/* hw/hw_q4r4.h:22-33 -- IEEE half to float, subnormals normalised. */
ORACLE_API float oracle_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h >> 15) << 31;
    int exp = (h >> 10) & 31;
    uint32_t man = h & 1023u;
    uint32_t bits;
    if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else if (exp != 0) {
        bits = sign | ((uint32_t)(exp + 112) << 23) | (man << 13);
    } else if (man == 0) {
        bits = sign;
    } else {
        int e = 113;                         /* value = man * 2^-24 */
        while (!(man & 1024u)) { man <<= 1; e--; }
        bits = sign | ((uint32_t)e << 23) | ((man & 1023u) << 13);
    }
    float f; memcpy(&f, &bits, 4); return f;
}

/* nn/quant.c:110-126 -- float to IEEE half, round to nearest even. */
ORACLE_API uint16_t oracle_f32_to_f16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    uint32_t e8 = (u >> 23) & 255u, man = u & 0x7fffffu;
    if (e8 == 255u) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u : 0u));
    int e = (int)e8 - 112;                   /* re-biased half exponent */
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return sign;
        uint32_t full = man | 0x800000u;
        int drop = 14 - e;
        uint32_t q = full >> drop, rest = full & ((1u << drop) - 1u), mid = 1u << (drop - 1);
        if (rest > mid || (rest == mid && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)e << 10) | (man >> 13), rest = man & 0x1fffu;
    if (rest > 0x1000u || (rest == 0x1000u && (q & 1u))) q++;
    return (uint16_t)(sign | q);
}

/* ------------------------------------------------------------------ */
/* activation quantizers                                               */
/* ------------------------------------------------------------------ */

/* hw/hw_quant.h:9-16 -- per-row symmetric int8; returns the scale.
 * No clamp: |q| <= 127 follows from s >= amax/127. */
ORACLE_API float oracle_qrow_i8(const float *x, int8_t *q, int n) {
    float amax = 0.f;
    for (int i = 0; i < n; i++) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    float s = amax / 127.f;
    if (s < 1e-12f) s = 1e-12f;
    float inv = 1.f / s;
    for (int i = 0; i < n; i++) q[i] = (int8_t)lrintf(x[i] * inv);
    return s;
}

/* hw/hw_q4r4.h:36-45 -- per group of 32: int8 codes, f32 scale, int32 code sum. */
ORACLE_API void oracle_quant_g32(const float *x, int I, int8_t *xq, float *xs, int32_t *xsum) {
    for (int g = 0; g < I / 32; g++) {
        const float *p = x + 32 * g;
        float amax = 0.f;
        for (int j = 0; j < 32; j++) { float a = fabsf(p[j]); if (a > amax) amax = a; }
        float s = amax / 127.f;
        if (s < 1e-30f) s = 1e-30f;
        float inv = 1.f / s;
        int32_t total = 0;
        for (int j = 0; j < 32; j++) {
            int v = (int)lrintf(p[j] * inv);
            xq[32 * g + j] = (int8_t)v;
            total += v;
        }
        xs[g] = s; xsum[g] = total;
    }
}

/* ------------------------------------------------------------------ */
/* integer dots                                                        */
/* ------------------------------------------------------------------ */

/* hw/hw_scalar.h:8-12 -- the contract every SIMD tier must match exactly. */
ORACLE_API int32_t oracle_dot_i8i8(const int8_t *w, const int8_t *x, int n) {
    int32_t acc = 0;
    for (int i = 0; i < n; i++) acc += (int32_t)w[i] * (int32_t)x[i];
    return acc;
}

/* hw/hw_scalar.h:14-22 -- per-row int4: element 2k in the low nibble, 2k+1 in
 * the high nibble, stored code = value + 8. */
ORACLE_API int32_t oracle_dot_i4i8(const uint8_t *w4, const int8_t *x, int n) {
    int32_t acc = 0;
    for (int i = 0; i < n; i++) {
        int nib = (i & 1) ? (w4[i >> 1] >> 4) : (w4[i >> 1] & 15);
        acc += (nib - 8) * (int32_t)x[i];
    }
    return acc;
}

/* ------------------------------------------------------------------ */
/* Q8_0 driver                                                         */
/* ------------------------------------------------------------------ */

/* nn/matmul.c:29-36,51-66 (IDOT=1 path): quantize each activation row, then
 * y[s][o] = (scale[o] * sx[s]) * (float)dot.  acc32 (optional) receives the
 * int32 accumulators [S][O]; xi_out/sx_out (optional) the quantized rows. */
ORACLE_API void oracle_matmul_q_s(float *y, const float *x, const int8_t *q, const float *scale,
                                  int S, int I, int O, int32_t *acc32, int8_t *xi_out, float *sx_out) {
    int8_t *xi = xi_out ? xi_out : (int8_t *)malloc((size_t)S * I + 1);
    float *sx = sx_out ? sx_out : (float *)malloc(sizeof(float) * (S ? S : 1));
    for (int s = 0; s < S; s++) sx[s] = oracle_qrow_i8(x + (size_t)s * I, xi + (size_t)s * I, I);
    #pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const int8_t *w = q + (size_t)o * I;
        for (int s = 0; s < S; s++) {
            int32_t d = oracle_dot_i8i8(w, xi + (size_t)s * I, I);
            if (acc32) acc32[(size_t)s * O + o] = d;
            y[(size_t)s * O + o] = scale[o] * sx[s] * (float)d;
        }
    }
    if (!xi_out) free(xi);
    if (!sx_out) free(sx);
}

/* nn/matmul.c:75-96,98-106 with IDOT4=1: per-row int4 weights, int8 activations. */
ORACLE_API void oracle_matmul_i4_idot_s(float *y, const float *x, const uint8_t *q4, const float *scale,
                                        int S, int I, int O) {
    int8_t *xi = (int8_t *)malloc((size_t)S * I + 1);
    float *sx = (float *)malloc(sizeof(float) * (S ? S : 1));
    int rb = (I + 1) / 2;
    for (int s = 0; s < S; s++) sx[s] = oracle_qrow_i8(x + (size_t)s * I, xi + (size_t)s * I, I);
    #pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++)
        for (int s = 0; s < S; s++)
            y[(size_t)s * O + o] = scale[o] * sx[s] *
                (float)oracle_dot_i4i8(q4 + (size_t)o * rb, xi + (size_t)s * I, I);
    free(xi); free(sx);
}

/* nn/quant.c:57-83 -- grouped int4 (WF_I4G): per row and group of gs weights the
 * scale is amax/7 floored at 1e-8, code = clamp(lrintf(w/s), -8, 7) + 8, the even
 * element in the low nibble.  Row o: (I+1)/2 bytes, scales [O][ceil(I/gs)] f32. */
ORACLE_API void oracle_pack_int4_grouped(const float *w, uint8_t *q4, float *scale, int O, int I, int gs) {
    int rb = (I + 1) / 2, ng = (I + gs - 1) / gs;
    for (int o = 0; o < O; o++) {
        const float *wr = w + (size_t)o * I;
        for (int g = 0; g * gs < I; g++) {
            int base = g * gs, glen = gs;
            if (base + glen > I) glen = I - base;
            float amax = 0.f;
            for (int i = base; i < base + glen; i++) { float a = fabsf(wr[i]); if (a > amax) amax = a; }
            float sc = amax / 7.f;
            if (sc < 1e-8f) sc = 1e-8f;
            scale[(size_t)o * ng + g] = sc;
            for (int i = base; i < base + glen; i += 2) {
                int v0 = (int)lrintf(wr[i] / sc), v1 = 0;
                if (v0 > 7) v0 = 7;
                if (v0 < -8) v0 = -8;
                if (i + 1 < base + glen) {
                    v1 = (int)lrintf(wr[i + 1] / sc);
                    if (v1 > 7) v1 = 7;
                    if (v1 < -8) v1 = -8;
                }
                q4[(size_t)o * rb + (i >> 1)] = (uint8_t)((v0 + 8) | ((v1 + 8) << 4));
            }
        }
    }
}

/* nn/matmul.c:164-197 with IDOT4=1 and gs = 32 (the integer path of WF_I4G): the
 * activation row is quantized per ROW (qrow_i8); per group the integer sum of
 * (nibble - 8) * x is exact (hw/hw_quant.h:35-50; the AVX512-VNNI kernel
 * hw/hw_avx512.h:155-176 computes the same integers as sum(nibble * x) - 8 * xgsum);
 * one f32 term per group is added in ascending group order, acc += scl[g] * (float)d,
 * which the reference's builds contract into a fused multiply-add (gcc -O2 keeps
 * -ffp-contract=fast and both of its x86 tiers have FMA); the result is sx * acc. */
ORACLE_API void oracle_matmul_i4g_idot_s(float *y, const float *x, const uint8_t *q4, const float *scale,
                                         int S, int I, int O) {
    int8_t *xi = (int8_t *)malloc((size_t)S * I + 1);
    float *sx = (float *)malloc(sizeof(float) * (S ? S : 1));
    int rb = (I + 1) / 2, ng = I / 32;
    for (int s = 0; s < S; s++) sx[s] = oracle_qrow_i8(x + (size_t)s * I, xi + (size_t)s * I, I);
    #pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w4 = q4 + (size_t)o * rb;
        const float *scl = scale + (size_t)o * ng;
        for (int s = 0; s < S; s++) {
            const int8_t *xr = xi + (size_t)s * I;
            float acc = 0.f;
            for (int g = 0; g < ng; g++) {
                int32_t d = 0;
                for (int j = 0; j < 32; j++) {
                    int e = g * 32 + j;
                    uint8_t b = w4[e >> 1];
                    int v = (e & 1) ? (b >> 4) : (b & 0xF);
                    d += (v - 8) * xr[e];
                }
                acc = fmaf(scl[g], (float)d, acc);
            }
            y[(size_t)s * O + o] = sx[s] * acc;
        }
    }
    free(xi); free(sx);
}

/* The same layout through the reference's DEFAULT product (no IDOT4): f32 activations x dequantized int4, one scale
 * multiply per group (i4g_f32_rows, nn/matmul.c:196-253): a += (sum_j x[j] * (float)(nibble_j - 8)) * scl[g] in
 * ascending group order.  The sum inside a group is taken here in element order; the reference's SIMD tiers take it in
 * their own lane orders, so this restatement agrees with the compiled reference to f32 rounding, not bit for bit. */
ORACLE_API void oracle_matmul_i4g_f32_s(float *y, const float *x, const uint8_t *q4, const float *scale,
                                        int S, int I, int O) {
    int rb = (I + 1) / 2, ng = (I + 31) / 32;
    #pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const uint8_t *w4 = q4 + (size_t)o * rb;
        const float *scl = scale + (size_t)o * ng;
        for (int s = 0; s < S; s++) {
            const float *xs = x + (size_t)s * I;
            float a = 0.f;
            for (int g = 0; g < ng; g++) {
                float p = 0.f;
                for (int e = g * 32; e < g * 32 + 32 && e < I; e++) {
                    uint8_t b = w4[e >> 1];
                    int v = (e & 1) ? (b >> 4) : (b & 0xF);
                    p += xs[e] * (float)(v - 8);
                }
                a += p * scl[g];
            }
            y[(size_t)s * O + o] = a;
        }
    }
}

/* ------------------------------------------------------------------ */
/* Q4R4: 4-row blocks, groups of 32, f16 scale stream                  */
/* ------------------------------------------------------------------ */

/* Integer part shared by both kernels below: for block row r and group g,
 * sum over j<16 of low_nibble(byte j) * x[j] + high_nibble(byte j) * x[j+16]
 * (hw/hw_q4r4.h:56-57).  The codes are unsigned 0..15. */
static int32_t q4r4_group_dot(const uint8_t *row16, const int8_t *xg) {
    int32_t acc = 0;
    for (int j = 0; j < 16; j++)
        acc += (int32_t)(row16[j] & 15) * xg[j] + (int32_t)(row16[j] >> 4) * xg[j + 16];
    return acc;
}

/* hw/hw_q4r4.h:47-63 -- one 4-row block against ns token rows; the offset -8
 * is removed in the integer domain, then one fused multiply-add per group in
 * ascending group order.  isum (optional) gets the offset-corrected int32 group
 * sums laid out [t][r][g]. */
ORACLE_API void oracle_q4r4_gemm(const uint8_t *w, const uint16_t *d, const int8_t *xq, const float *xs,
                                 const int32_t *xsum, int nb, int ns, float *y, int ys, int32_t *isum) {
    int I = nb * 32;
    for (int t = 0; t < ns; t++)
        for (int r = 0; r < 4; r++) {
            float acc = 0.f;
            for (int g = 0; g < nb; g++) {
                int32_t s = q4r4_group_dot(w + (size_t)g * 64 + r * 16, xq + (size_t)t * I + g * 32)
                            - 8 * xsum[(size_t)t * nb + g];
                if (isum) isum[((size_t)t * 4 + r) * nb + g] = s;
                float c = oracle_f16_to_f32(d[(size_t)g * 4 + r]) * xs[(size_t)t * nb + g];
                acc = fmaf((float)s, c, acc);
            }
            y[(size_t)t * ys + r] = acc;
        }
}

/* hw/hw_q4r4.h:86-93 -- scales of four token rows re-laid per group:
 * xst[g*4+t] = xs[t][g], xct[g*4+t] = 8 * xsum[t][g] * xs[t][g] (left to right). */
ORACLE_API void oracle_q4r4_tile_scales(const float *xs, const int32_t *xsum, int nb, float *xst, float *xct) {
    for (int g = 0; g < nb; g++)
        for (int t = 0; t < 4; t++) {
            float s = xs[(size_t)t * nb + g];
            xst[g * 4 + t] = s;
            xct[g * 4 + t] = 8.f * (float)xsum[(size_t)t * nb + g] * s;
        }
}

/* hw/hw_q4r4.h:69-84 -- the 4-token prefill tile: the raw (uncorrected) int
 * sum is scaled first, then the offset term is subtracted in float. */
ORACLE_API void oracle_q4r4_gemm4t(const uint8_t *w, const uint16_t *d, const int8_t *xq, int64_t ldx,
                                   const float *xst, const float *xct, int nb, float *y, int ys) {
    for (int t = 0; t < 4; t++)
        for (int r = 0; r < 4; r++) {
            float acc = 0.f;
            for (int g = 0; g < nb; g++) {
                int32_t s = q4r4_group_dot(w + (size_t)g * 64 + r * 16, xq + t * ldx + g * 32);
                float dd = oracle_f16_to_f32(d[(size_t)g * 4 + r]);
                acc = fmaf((float)s, dd * xst[g * 4 + t], acc);
                acc = fmaf(-dd, xct[g * 4 + t], acc);
            }
            y[(size_t)t * ys + r] = acc;
        }
}

/* nn/matmul.c:371-433 -- the driver: group-quantize the S rows; tokens are cut
 * into tiles of 32; inside a tile every complete group of 4 tokens goes through
 * the 4-token kernel and the remaining (tile size % 4) tokens through the
 * token-by-token kernel.  Which kernel a token meets decides how the -8 offset
 * is folded, so the split must be reproduced to match bit for bit. */
ORACLE_API void oracle_matmul_q4r4_s(float *y, const float *x, const uint8_t *q4, const uint16_t *s16,
                                     int S, int I, int O) {
    int nb = I / 32, nblk = (O + 3) / 4, full = O / 4;
    size_t SI = (size_t)S * I + 1, SN = (size_t)S * nb + 1;
    int8_t *xq = (int8_t *)malloc(SI);
    float *xs = (float *)malloc(SN * 4), *xst = (float *)malloc(SN * 4), *xct = (float *)malloc(SN * 4);
    int32_t *xsum = (int32_t *)malloc(SN * 4);
    for (int s = 0; s < S; s++)
        oracle_quant_g32(x + (size_t)s * I, I, xq + (size_t)s * I, xs + (size_t)s * nb, xsum + (size_t)s * nb);
    for (int k = 0; k < S / 4; k++)
        oracle_q4r4_tile_scales(xs + (size_t)k * 4 * nb, xsum + (size_t)k * 4 * nb, nb,
                                xst + (size_t)k * nb * 4, xct + (size_t)k * nb * 4);
    for (int t0 = 0; t0 < S; t0 += 32) {
        int ns = S - t0 < 32 ? S - t0 : 32, n4 = ns / 4 * 4;
        #pragma omp parallel for schedule(dynamic, 8)
        for (int ob = 0; ob < nblk; ob++) {
            float tmp[4 * 32];
            int ragged = (ob == full);
            float *yo = ragged ? tmp : y + (size_t)t0 * O + ob * 4;
            int ys = ragged ? 4 : O;
            const uint8_t *wb = q4 + (size_t)ob * nb * 64;
            const uint16_t *db = s16 + (size_t)ob * nb * 4;
            for (int t = 0; t < n4; t += 4)
                oracle_q4r4_gemm4t(wb, db, xq + (size_t)(t0 + t) * I, I,
                                   xst + (size_t)((t0 + t) / 4) * nb * 4, xct + (size_t)((t0 + t) / 4) * nb * 4,
                                   nb, yo + (size_t)t * ys, ys);
            if (n4 < ns)
                oracle_q4r4_gemm(wb, db, xq + (size_t)(t0 + n4) * I, xs + (size_t)(t0 + n4) * nb,
                                 xsum + (size_t)(t0 + n4) * nb, nb, ns - n4, yo + (size_t)n4 * ys, ys, NULL);
            if (ragged)
                for (int t = 0; t < ns; t++)
                    for (int r = 0; r < O - full * 4; r++)
                        y[(size_t)(t0 + t) * O + full * 4 + r] = tmp[t * 4 + r];
        }
    }
    free(xq); free(xs); free(xst); free(xct); free(xsum);
}

/* ------------------------------------------------------------------ */
/* load-time weight quantizers                                         */
/* ------------------------------------------------------------------ */

/* nn/quant.c:12-33 -- per-row int8 (bits=8) with a true division per element. */
ORACLE_API void oracle_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I, int bits) {
    int qmax = (1 << (bits - 1)) - 1;
    #pragma omp parallel for schedule(static)
    for (int o = 0; o < O; o++) {
        const float *row = w + (size_t)o * I;
        float amax = 0.f;
        for (int i = 0; i < I; i++) { float a = fabsf(row[i]); if (a > amax) amax = a; }
        float s = amax / (float)qmax;
        if (s < 1e-8f) s = 1e-8f;
        scale[o] = s;
        for (int i = 0; i < I; i++) {
            int v = (int)lrintf(row[i] / s);
            if (v > qmax) v = qmax;
            if (v < -qmax - 1) v = -qmax - 1;
            q[(size_t)o * I + i] = (int8_t)v;
        }
    }
}

/* nn/quant.c:35-55 -- per-row int4, scale amax/7, code = clamp(round(w/s),-8,7)+8. */
ORACLE_API void oracle_pack_int4(const float *w, uint8_t *q4, float *scale, int O, int I) {
    int rb = (I + 1) / 2;
    for (int o = 0; o < O; o++) {
        const float *row = w + (size_t)o * I;
        float amax = 0.f;
        for (int i = 0; i < I; i++) { float a = fabsf(row[i]); if (a > amax) amax = a; }
        float s = amax / 7.f;
        if (s < 1e-8f) s = 1e-8f;
        scale[o] = s;
        for (int b = 0; b < rb; b++) {
            int code[2] = { 8, 8 };
            for (int h = 0; h < 2; h++) {
                int i = 2 * b + h;
                if (i >= I) break;
                int v = (int)lrintf(row[i] / s);
                if (v > 7) v = 7;
                if (v < -8) v = -8;
                code[h] = v + 8;
            }
            q4[(size_t)o * rb + b] = (uint8_t)(code[0] | (code[1] << 4));
        }
    }
}

/* nn/quant.c:157-179 -- one 4-row Q4R4 block.  Group scale: the largest-
 * magnitude weight maps to code -8 unless that step would clip the largest
 * weight of the other sign; the scale is stored signed in f16 and the codes are
 * computed from the ROUNDED scale.  Byte j of a row = code[j] | code[j+16] << 4.
 * Rows past nr: bytes 0x88 (code 8 = value 0), scale bits 0. */
ORACLE_API void oracle_pack_q4r4_block(const float *w, int nr, int I, uint8_t *blk, uint16_t *d) {
    int nb = I / 32;
    for (int g = 0; g < nb; g++)
        for (int r = 0; r < 4; r++) {
            uint8_t *out = blk + (size_t)g * 64 + r * 16;
            if (r >= nr) { memset(out, 0x88, 16); d[(size_t)g * 4 + r] = 0; continue; }
            const float *p = w + (size_t)r * I + g * 32;
            float big = 0.f;
            for (int j = 0; j < 32; j++) if (fabsf(p[j]) > fabsf(big)) big = p[j];
            float other = 0.f;
            for (int j = 0; j < 32; j++)
                if ((p[j] > 0) != (big > 0) && fabsf(p[j]) > other) other = fabsf(p[j]);
            float step = fmaxf(fabsf(big) / 8.f, other / 7.f);
            uint16_t h = oracle_f32_to_f16(big > 0 ? -step : step);
            float dd = oracle_f16_to_f32(h);
            float inv = dd != 0.f ? 1.f / dd : 0.f;
            uint8_t code[32];
            for (int j = 0; j < 32; j++) {
                int v = (int)lrintf(p[j] * inv);
                if (v < -8) v = -8;
                if (v > 7) v = 7;
                code[j] = (uint8_t)(v + 8);
            }
            d[(size_t)g * 4 + r] = h;
            for (int j = 0; j < 16; j++) out[j] = (uint8_t)(code[j] | (code[j + 16] << 4));
        }
}

/* runtime/rt_model_load.h:85-121 (r4_pack_part) -- a whole [O][I] matrix in
 * blocks of 4 rows; the last block may hold fewer than 4 rows. */
/* ---------------------------------------------------------------------------
 * Q8R4, the int8 sibling of Q4R4 (hw/hw_q4r4.h:92-130, nn/matmul.c:435-461,
 * nn/quant.c:135-155): the same 4-row blocks, groups of 32 and f16 scale stream, 128 bytes
 * per (block, group) = 4 rows x 32 signed codes, no offset term.  The single-token and the
 * 4-token kernels of the reference compute the same thing per (row, token):
 *   acc = fma((float)sum_g, f16(d[g][r]) * xs[t][g], acc), groups ascending
 * (the compiler contracts the reference's acc += a * b; spelled out here).
 * ------------------------------------------------------------------------- */
ORACLE_API void oracle_matmul_q8r4_s(float *y, const float *x, const int8_t *q8, const uint16_t *s16,
                                     int S, int I, int O) {
    int nb = I / 32, nblk = (O + 3) / 4;
    int8_t *xq = (int8_t *)malloc((size_t)S * I + 1);
    float *xs = (float *)malloc(((size_t)S * nb + 1) * 4);
    int32_t *xsum = (int32_t *)malloc(((size_t)S * nb + 1) * 4);
    for (int s = 0; s < S; s++)
        oracle_quant_g32(x + (size_t)s * I, I, xq + (size_t)s * I, xs + (size_t)s * nb, xsum + (size_t)s * nb);
    #pragma omp parallel for schedule(dynamic, 8)
    for (int ob = 0; ob < nblk; ob++) {
        const int8_t *wb = q8 + (size_t)ob * nb * 128;
        const uint16_t *db = s16 + (size_t)ob * nb * 4;
        for (int t = 0; t < S; t++)
            for (int r = 0; r < 4; r++) {
                if (ob * 4 + r >= O) continue;
                float acc = 0.f;
                for (int g = 0; g < nb; g++) {
                    const int8_t *wr = wb + (size_t)g * 128 + r * 32, *xg = xq + (size_t)t * I + g * 32;
                    int32_t sum = 0;
                    for (int j = 0; j < 32; j++) sum += (int32_t)wr[j] * xg[j];
                    acc = fmaf((float)sum, oracle_f16_to_f32(db[(size_t)g * 4 + r]) * xs[(size_t)t * nb + g], acc);
                }
                y[(size_t)t * O + ob * 4 + r] = acc;
            }
    }
    free(xq); free(xs); free(xsum);
}

ORACLE_API void oracle_pack_q8r4_block(const float *w, int nr, int I, int8_t *blk, uint16_t *d) {
    int nb = I / 32;
    for (int g = 0; g < nb; g++)
        for (int r = 0; r < 4; r++) {
            int8_t *out = blk + (size_t)g * 128 + r * 32;
            if (r >= nr) { memset(out, 0, 32); d[(size_t)g * 4 + r] = 0; continue; }
            const float *p = w + (size_t)r * I + g * 32;
            float big = 0.f;
            for (int j = 0; j < 32; j++) if (fabsf(p[j]) > fabsf(big)) big = p[j];
            float other = 0.f;
            for (int j = 0; j < 32; j++)
                if ((p[j] > 0) != (big > 0) && fabsf(p[j]) > other) other = fabsf(p[j]);
            float step = fmaxf(fabsf(big) / 128.f, other / 127.f);
            uint16_t h = oracle_f32_to_f16(big > 0 ? -step : step);
            float dd = oracle_f16_to_f32(h);
            float inv = dd != 0.f ? 1.f / dd : 0.f;
            for (int j = 0; j < 32; j++) {
                int v = (int)lrintf(p[j] * inv);
                if (v < -128) v = -128;
                if (v > 127) v = 127;
                out[j] = (int8_t)v;
            }
            d[(size_t)g * 4 + r] = h;
        }
}

ORACLE_API void oracle_pack_q8r4(const float *w, int O, int I, int8_t *q8, uint16_t *s16) {
    int nb = I / 32, nblk = (O + 3) / 4;
    #pragma omp parallel for schedule(static)
    for (int b = 0; b < nblk; b++) {
        int nr = O - 4 * b < 4 ? O - 4 * b : 4;
        oracle_pack_q8r4_block(w + (size_t)b * 4 * I, nr, I, q8 + (size_t)b * nb * 128, s16 + (size_t)b * nb * 4);
    }
}

ORACLE_API void oracle_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16) {
    int nb = I / 32, nblk = (O + 3) / 4;
    #pragma omp parallel for schedule(static)
    for (int b = 0; b < nblk; b++) {
        int nr = O - 4 * b < 4 ? O - 4 * b : 4;
        oracle_pack_q4r4_block(w + (size_t)b * 4 * I, nr, I, q4 + (size_t)b * nb * 64, s16 + (size_t)b * nb * 4);
    }
}

/* ------------------------------------------------------------------ */
/* expf                                                                 */
/* ------------------------------------------------------------------ */

/* The reference's SiLU, router softmax and output gate call the C library's expf
 * (hw/hw_ops.h:19-26, nn/moe.c:11,120,197, nn/attn.c:69).  That function is not
 * part of the reference tree: it is glibc's (2.39 in this image), whose algorithm
 * since 2.27 is the published table-driven one of ARM's optimized routines:
 *   z = x * 32/ln2,  k = round-to-nearest(z) taken by adding 1.5*2^52,  r = z - k,
 *   s = 2^(k/32): a 32-entry table of 2^(i/32) plus k/32 in the exponent field,
 *   exp(x) = s * (C0 r^3 + C1 r^2 + C2 r + 1), all in f64, rounded once to f32.
 * x86-64 machines with FMA run the build of it in which the compiler contracted
 * the multiply-adds: r = fma(32/ln2, x, -k), and the three polynomial steps as
 * written below.  This restatement equals the host's expf on every one of the
 * 2^32 float inputs (oracle_expf_mismatches over the full range; the test-suite
 * checks a sample in each run).  Table entry i = bits(2^(i/32) rounded to nearest
 * f64) - (i << 47); tests/test_oracle.py recomputes the entries at high precision. */
static const uint64_t oracle_exp2_tab[32] = {
    0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL,
    0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL,
    0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL,
    0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL,
    0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL,
    0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL,
    0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL,
    0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL};

ORACLE_API uint64_t oracle_exp2_tab_entry(int i) { return oracle_exp2_tab[i & 31]; }

ORACLE_API float oracle_expf(float x) {
    uint32_t ux; memcpy(&ux, &x, 4);
    const uint32_t top = (ux >> 20) & 0x7ffu;
    if (top >= 0x42bu) {                          /* |x| >= 88, infinities, NaN */
        if (ux == 0xff800000u) return 0.f;
        if (top >= 0x7f8u) return x + x;
        if (x > 0x1.62e42ep6f) return INFINITY;
        if (x < -0x1.9fe368p6f) return 0.f;
    }
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
    const double c0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, c1 = 0x1.ebfce50fac4f3p-3 / 32 / 32,
                 c2 = 0x1.62e42ff0c52d6p-1 / 32;
    const double shift = 0x1.8p52;
    const double xd = (double)x;
    const double z = inv_ln2_n * xd;
    double kd = z + shift;
    uint64_t ki; memcpy(&ki, &kd, 8);
    kd -= shift;
    const double r = fma(inv_ln2_n, xd, -kd);
    const uint64_t sb = oracle_exp2_tab[ki & 31] + (ki << 47);
    double s; memcpy(&s, &sb, 8);
    const double p = fma(c0, r, c1);
    const double r2 = r * r;
    double y = fma(c2, r, 1.0);
    y = fma(p, r2, y);
    return (float)(y * s);
}

/* How many of the float bit patterns first, first+stride, ... (< first + count*stride,
 * NaNs skipped) give different bits from the host C library's expf. */
ORACLE_API int64_t oracle_expf_mismatches(uint32_t first, uint32_t stride, int64_t count) {
    int64_t bad = 0;
    #pragma omp parallel for reduction(+:bad) schedule(static)
    for (int64_t j = 0; j < count; j++) {
        uint32_t u = first + (uint32_t)j * stride;
        float x; memcpy(&x, &u, 4);
        if (x != x) continue;
        float a = expf(x), b = oracle_expf(x);
        uint32_t ua, ub; memcpy(&ua, &a, 4); memcpy(&ub, &b, 4);
        if (ua != ub) bad++;
    }
    return bad;
}

/* ------------------------------------------------------------------ */
/* router                                                              */
/* ------------------------------------------------------------------ */

/* hw/hw_ops.h:22-26 -- in-place softmax: max from -1e30, expf (restated above), sequential
 * f32 sum, one division per element. */
ORACLE_API void oracle_softmax(float *x, int n) {
    float m = -1e30f;
    for (int i = 0; i < n; i++) if (x[i] > m) m = x[i];
    float total = 0.f;
    for (int i = 0; i < n; i++) { x[i] = oracle_expf(x[i] - m); total += x[i]; }
    for (int i = 0; i < n; i++) x[i] /= total;
}

/* runtime/moecache.c:97-111 -- K rounds of "largest not yet taken", strict >
 * from a floor of -1e30 so ties resolve to the lowest index; optional
 * renormalisation by the sequential sum of the K picked values. */
ORACLE_API void oracle_moe_topk(const float *p, int E, int K, int *idx, float *w, int norm_topk) {
    for (int k = 0; k < K; k++) {
        int best = -1; float bv = -1e30f;
        for (int e = 0; e < E; e++) {
            int used = 0;
            for (int j = 0; j < k; j++) if (idx[j] == e) { used = 1; break; }
            if (!used && p[e] > bv) { bv = p[e]; best = e; }
        }
        idx[k] = best; w[k] = bv;
    }
    if (norm_topk) {
        float total = 0.f;
        for (int k = 0; k < K; k++) total += w[k];
        if (total > 0) for (int k = 0; k < K; k++) w[k] /= total;
    }
}

/* nn/moe.c:27-30 -- softmax in place, then top-K with renormalisation on. */
ORACLE_API void oracle_route_topk(float *logits, int E, int K, int *idx, float *w) {
    oracle_softmax(logits, E);
    oracle_moe_topk(logits, E, K, idx, w, 1);
}

/* nn/moe.c:10-25 -- the LFM2 gate: probs = sigmoid(logit) with the C library's expf; K rounds of "largest
 * probs + bias not yet taken" (strict > from -1e30: ties to the lowest index); the weights are the
 * UNBIASED probabilities of the picks, divided by their sequential sum when that is positive. */
ORACLE_API void oracle_route_sigmoid(const float *lb, const float *bias, int E, int K, int *idx, float *w) {
    float *probs = (float *)malloc(sizeof(float) * (size_t)E);
    for (int e = 0; e < E; e++) probs[e] = 1.f / (1.f + oracle_expf(-lb[e]));
    for (int k = 0; k < K; k++) {
        int best = -1; float bv = -1e30f;
        for (int e = 0; e < E; e++) {
            float v = probs[e] + (bias ? bias[e] : 0.f);
            int used = 0;
            for (int j = 0; j < k; j++) if (idx[j] == e) used = 1;
            if (!used && v > bv) { bv = v; best = e; }
        }
        idx[k] = best;
    }
    float ws = 0.f;
    for (int k = 0; k < K; k++) { w[k] = probs[idx[k]]; ws += w[k]; }
    if (ws > 0) for (int k = 0; k < K; k++) w[k] /= ws;
    free(probs);
}

/* nn/sample.c:9-13 -- greedy token: first index of the maximum. */
ORACLE_API int oracle_argmax(const float *v, int n) {
    int best = 0; float bv = v[0];
    for (int i = 1; i < n; i++) if (v[i] > bv) { bv = v[i]; best = i; }
    return best;
}

/* ------------------------------------------------------------------ */
/* activations and FFN / MoE blocks                                    */
/* ------------------------------------------------------------------ */

/* hw/hw_ops.h:19-21 -- g = silu(g) * u, silu(v) = v / (1 + expf(-v)). */
ORACLE_API void oracle_silu_mul(float *g, const float *u, int64_t n) {
    for (int64_t i = 0; i < n; i++) { float v = g[i]; g[i] = (v / (1.f + oracle_expf(-v))) * u[i]; }
}

/* engines/gemma.c:389-391,398 -- g = gelu_tanh(g) * u. */
ORACLE_API void oracle_gelu_mul(float *g, const float *u, int64_t n) {
    for (int64_t i = 0; i < n; i++) {
        float v = g[i];
        /* gcc fuses `v + (0.044715f*v*v)*v` into one multiply-add in the reference build */
        float t = 0.5f * v * (1.f + tanhf(0.7978845608028654f * fmaf(0.044715f * v * v, v, v)));
        g[i] = t * u[i];
    }
}

/* nn/ffn.c:26-55, engines/qwen.c:654-679, engines/gemma.c:392-401 with Q8_0
 * matrices: gate and up GEMV/GEMM, activation * up, down GEMV/GEMM.
 * act: 0 = SiLU (qwen), 1 = tanh-GeLU (gemma).  h_out (optional) gets the
 * [S][I] activation fed to the down projection. */
ORACLE_API void oracle_ffn_q8(float *out, const float *x, int S, int D, int I, int act,
                              const int8_t *gq, const float *gs, const int8_t *uq, const float *us,
                              const int8_t *dq, const float *ds, float *h_out) {
    size_t n = (size_t)S * I + 1;
    float *g = h_out ? h_out : (float *)malloc(n * 4), *u = (float *)malloc(n * 4);
    oracle_matmul_q_s(g, x, gq, gs, S, D, I, NULL, NULL, NULL);
    oracle_matmul_q_s(u, x, uq, us, S, D, I, NULL, NULL, NULL);
    if (act == 0) oracle_silu_mul(g, u, (int64_t)S * I); else oracle_gelu_mul(g, u, (int64_t)S * I);
    oracle_matmul_q_s(out, g, dq, ds, S, I, D, NULL, NULL, NULL);
    if (!h_out) free(g);
    free(u);
}

/* Same block with Q4R4 matrices (what QBITS=4 Q4FMT=r4 loads). */
ORACLE_API void oracle_ffn_q4r4(float *out, const float *x, int S, int D, int I, int act,
                                const uint8_t *gq, const uint16_t *gs, const uint8_t *uq, const uint16_t *us,
                                const uint8_t *dq, const uint16_t *ds) {
    size_t n = (size_t)S * I + 1;
    float *g = (float *)malloc(n * 4), *u = (float *)malloc(n * 4);
    oracle_matmul_q4r4_s(g, x, gq, gs, S, D, I);
    oracle_matmul_q4r4_s(u, x, uq, us, S, D, I);
    if (act == 0) oracle_silu_mul(g, u, (int64_t)S * I); else oracle_gelu_mul(g, u, (int64_t)S * I);
    oracle_matmul_q4r4_s(out, g, dq, ds, S, I, D);
    free(g); free(u);
}

/* Experts of one MoE layer, all resident, per-row int8 (the layout of
 * runtime/moe.h:35-39 ExpertSlot, one slot per expert id):
 *   g,u: [E][I][D] int8, gs,us: [E][I] f32;  d: [E][D][I] int8, ds: [E][D] f32. */
typedef struct {
    int E, K, I, D;
    const int8_t *g, *u, *d;
    const float *gs, *us, *ds;
} OracleExperts;

/* nn/moe.c:33-153 (softmax/top-k variant, int8 experts, no shared expert),
 * given the router logits of the one token: route, quantize x once, all gate
 * and up rows, SiLU*up then per-expert re-quantization, all down rows, and the
 * weighted sum accumulated in selection order k = 0..K-1 (one fused
 * multiply-add per element).  idx_out/w_out (optional) return the routing. */
static void moe_d1_impl(const OracleExperts *ex, const float *x, float *logits, float *out,
                        int *idx_out, float *w_out, int sig, const float *bias);
ORACLE_API void oracle_moe_d1(const OracleExperts *ex, const float *x, float *logits, float *out,
                              int *idx_out, float *w_out) {
    moe_d1_impl(ex, x, logits, out, idx_out, w_out, 0, NULL);
}
/* moty_nn_moe_sigmoid_d1 (nn/moe.c:154): the same block behind the sigmoid + bias gate */
ORACLE_API void oracle_moe_sigmoid_d1(const OracleExperts *ex, const float *x, float *logits, const float *bias, float *out,
                                      int *idx_out, float *w_out) {
    moe_d1_impl(ex, x, logits, out, idx_out, w_out, 1, bias);
}
static void moe_d1_impl(const OracleExperts *ex, const float *x, float *logits, float *out,
                        int *idx_out, float *w_out, int sig, const float *bias) {
    int E = ex->E, K = ex->K, I = ex->I, D = ex->D;
    int idx[64]; float w[64];
    if (sig) oracle_route_sigmoid(logits, bias, E, K, idx, w);
    else oracle_route_topk(logits, E, K, idx, w);
    int8_t *xi = (int8_t *)malloc(D), *hi = (int8_t *)malloc(I);
    float *gb = (float *)malloc((size_t)I * 4), *ub = (float *)malloc((size_t)I * 4), *hb = (float *)malloc((size_t)D * 4);
    float sx = oracle_qrow_i8(x, xi, D);
    memset(out, 0, (size_t)D * 4);
    /* the reference computes all experts' rows first and sums afterwards; the
     * per-expert values and the k-ordered accumulation are what matter */
    float *hall = (float *)malloc((size_t)K * D * 4);
    for (int k = 0; k < K; k++) {
        size_t e = (size_t)idx[k];
        #pragma omp parallel for schedule(static)
        for (int i = 0; i < I; i++) {
            gb[i] = ex->gs[e * I + i] * sx * (float)oracle_dot_i8i8(ex->g + (e * I + i) * D, xi, D);
            ub[i] = ex->us[e * I + i] * sx * (float)oracle_dot_i8i8(ex->u + (e * I + i) * D, xi, D);
        }
        oracle_silu_mul(gb, ub, I);
        float sh = oracle_qrow_i8(gb, hi, I);
        #pragma omp parallel for schedule(static)
        for (int dd = 0; dd < D; dd++)
            hall[(size_t)k * D + dd] = ex->ds[e * D + dd] * sh * (float)oracle_dot_i8i8(ex->d + (e * D + dd) * I, hi, I);
    }
    for (int k = 0; k < K; k++)
        for (int dd = 0; dd < D; dd++) out[dd] = fmaf(w[k], hall[(size_t)k * D + dd], out[dd]);
    if (idx_out) memcpy(idx_out, idx, sizeof(int) * K);
    if (w_out) memcpy(w_out, w, sizeof(float) * K);
    (void)hb;
    free(xi); free(hi); free(gb); free(ub); free(hb); free(hall);
}

/* nn/moe.c:159-205 (softmax/top-k, int8 experts, no shared expert), given the
 * router logits [S][E]: per-token routing, then experts in ascending id; each
 * expert gathers its tokens in ascending token order, runs the three Q8_0
 * matmuls on the gathered rows and scatter-adds weight * h.  A token's output
 * is therefore accumulated in ascending EXPERT order, unlike the S=1 path. */
static void moe_batch_impl(const OracleExperts *ex, const float *x, int S, float *logits, float *out,
                           int *idx_out, float *w_out, int sig, const float *bias);
ORACLE_API void oracle_moe_batch(const OracleExperts *ex, const float *x, int S, float *logits, float *out,
                                 int *idx_out, float *w_out) {
    moe_batch_impl(ex, x, S, logits, out, idx_out, w_out, 0, NULL);
}
/* moty_nn_moe_sigmoid_batch (nn/moe.c:207) */
ORACLE_API void oracle_moe_sigmoid_batch(const OracleExperts *ex, const float *x, int S, float *logits, const float *bias,
                                         float *out, int *idx_out, float *w_out) {
    moe_batch_impl(ex, x, S, logits, out, idx_out, w_out, 1, bias);
}
static void moe_batch_impl(const OracleExperts *ex, const float *x, int S, float *logits, float *out,
                           int *idx_out, float *w_out, int sig, const float *bias) {
    int E = ex->E, K = ex->K, I = ex->I, D = ex->D;
    int *idx = (int *)malloc(sizeof(int) * (size_t)S * K);
    float *rw = (float *)malloc(sizeof(float) * (size_t)S * K);
    for (int s = 0; s < S; s++) {
        if (sig) oracle_route_sigmoid(logits + (size_t)s * E, bias, E, K, idx + (size_t)s * K, rw + (size_t)s * K);
        else oracle_route_topk(logits + (size_t)s * E, E, K, idx + (size_t)s * K, rw + (size_t)s * K);
    }
    memset(out, 0, (size_t)S * D * 4);
    int *tl = (int *)malloc(sizeof(int) * (S ? S : 1));
    float *xsub = (float *)malloc((size_t)S * D * 4 + 4), *g = (float *)malloc((size_t)S * I * 4 + 4);
    float *u = (float *)malloc((size_t)S * I * 4 + 4), *h = (float *)malloc((size_t)S * D * 4 + 4);
    for (int e = 0; e < E; e++) {
        int nt = 0;
        for (int s = 0; s < S; s++)
            for (int k = 0; k < K; k++) if (idx[(size_t)s * K + k] == e) { tl[nt++] = s; break; }
        if (!nt) continue;
        for (int t = 0; t < nt; t++) memcpy(xsub + (size_t)t * D, x + (size_t)tl[t] * D, (size_t)D * 4);
        oracle_matmul_q_s(g, xsub, ex->g + (size_t)e * I * D, ex->gs + (size_t)e * I, nt, D, I, NULL, NULL, NULL);
        oracle_matmul_q_s(u, xsub, ex->u + (size_t)e * I * D, ex->us + (size_t)e * I, nt, D, I, NULL, NULL, NULL);
        oracle_silu_mul(g, u, (int64_t)nt * I);
        oracle_matmul_q_s(h, g, ex->d + (size_t)e * D * I, ex->ds + (size_t)e * D, nt, I, D, NULL, NULL, NULL);
        for (int t = 0; t < nt; t++)
            for (int k = 0; k < K; k++)
                if (idx[(size_t)tl[t] * K + k] == e) {
                    float wk = rw[(size_t)tl[t] * K + k];
                    float *o = out + (size_t)tl[t] * D;
                    for (int dd = 0; dd < D; dd++) o[dd] = fmaf(wk, h[(size_t)t * D + dd], o[dd]);
                }
    }
    if (idx_out) memcpy(idx_out, idx, sizeof(int) * (size_t)S * K);
    if (w_out) memcpy(w_out, rw, sizeof(float) * (size_t)S * K);
    free(idx); free(rw); free(tl); free(xsub); free(g); free(u); free(h);
}

/* engines/olmoe.c:219-244 -- OLMoE's own block: for every token, softmax +
 * top-K (renormalisation per config), then for each selected expert in
 * selection order three S=1 Q8_0 GEMVs and out += weight * h. */
ORACLE_API void oracle_olmoe_moe(const OracleExperts *ex, const float *x, int S, float *logits, float *out,
                                 int norm_topk, int *idx_out, float *w_out) {
    int E = ex->E, K = ex->K, I = ex->I, D = ex->D;
    float *g = (float *)malloc((size_t)I * 4), *u = (float *)malloc((size_t)I * 4), *h = (float *)malloc((size_t)D * 4);
    memset(out, 0, (size_t)S * D * 4);
    for (int s = 0; s < S; s++) {
        int idx[64]; float w[64];
        float *p = logits + (size_t)s * E;
        oracle_softmax(p, E);
        oracle_moe_topk(p, E, K, idx, w, norm_topk);
        const float *xs = x + (size_t)s * D;
        for (int k = 0; k < K; k++) {
            size_t e = (size_t)idx[k];
            oracle_matmul_q_s(g, xs, ex->g + e * I * D, ex->gs + e * I, 1, D, I, NULL, NULL, NULL);
            oracle_matmul_q_s(u, xs, ex->u + e * I * D, ex->us + e * I, 1, D, I, NULL, NULL, NULL);
            oracle_silu_mul(g, u, I);
            oracle_matmul_q_s(h, g, ex->d + e * D * I, ex->ds + e * D, 1, I, D, NULL, NULL, NULL);
            float *o = out + (size_t)s * D;
            for (int dd = 0; dd < D; dd++) o[dd] = fmaf(w[k], h[dd], o[dd]);
        }
        if (idx_out) memcpy(idx_out + (size_t)s * K, idx, sizeof(int) * K);
        if (w_out) memcpy(w_out + (size_t)s * K, w, sizeof(float) * K);
    }
    free(g); free(u); free(h);
}

/* Q4R4 experts (no reference engine stores experts this way; this is the
 * composition of reference functions the Qwen3-30B-A3B-shaped configuration
 * is checked against): routing as nn/moe.c:27-30, each expert's three
 * projections through the Q4R4 driver (nn/matmul.c:371-433) on its gathered
 * rows, accumulation order as nn/moe.c:200-202 (S>1) or :146-149 (S=1).
 *   g,u: [E] Q4R4 matrices of O=I rows, width D;  d: [E] Q4R4 of O=D, width I. */
typedef struct {
    int E, K, I, D;
    const uint8_t *g, *u, *d;        /* codes, expert-major */
    const uint16_t *gs, *us, *ds;    /* f16 scale streams, expert-major */
} OracleExpertsQ4;

ORACLE_API void oracle_moe_q4r4(const OracleExpertsQ4 *ex, const float *x, int S, float *logits, float *out,
                                int *idx_out, float *w_out) {
    int E = ex->E, K = ex->K, I = ex->I, D = ex->D;
    size_t gq = (size_t)((I + 3) / 4) * (D / 32) * 64, gsn = (size_t)((I + 3) / 4) * (D / 32) * 4;
    size_t dq = (size_t)((D + 3) / 4) * (I / 32) * 64, dsn = (size_t)((D + 3) / 4) * (I / 32) * 4;
    int *idx = (int *)malloc(sizeof(int) * (size_t)S * K);
    float *rw = (float *)malloc(sizeof(float) * (size_t)S * K);
    for (int s = 0; s < S; s++) oracle_route_topk(logits + (size_t)s * E, E, K, idx + (size_t)s * K, rw + (size_t)s * K);
    memset(out, 0, (size_t)S * D * 4);
    float *xsub = (float *)malloc((size_t)S * D * 4 + 4), *g = (float *)malloc((size_t)S * I * 4 + 4);
    float *u = (float *)malloc((size_t)S * I * 4 + 4), *h = (float *)malloc((size_t)S * D * 4 + 4);
    int *tl = (int *)malloc(sizeof(int) * (S ? S : 1));
    if (S == 1) {
        for (int k = 0; k < K; k++) {
            size_t e = (size_t)idx[k];
            oracle_matmul_q4r4_s(g, x, ex->g + e * gq, ex->gs + e * gsn, 1, D, I);
            oracle_matmul_q4r4_s(u, x, ex->u + e * gq, ex->us + e * gsn, 1, D, I);
            oracle_silu_mul(g, u, I);
            oracle_matmul_q4r4_s(h, g, ex->d + e * dq, ex->ds + e * dsn, 1, I, D);
            for (int dd = 0; dd < D; dd++) out[dd] = fmaf(rw[k], h[dd], out[dd]);
        }
    } else {
        for (int e = 0; e < E; e++) {
            int nt = 0;
            for (int s = 0; s < S; s++)
                for (int k = 0; k < K; k++) if (idx[(size_t)s * K + k] == e) { tl[nt++] = s; break; }
            if (!nt) continue;
            for (int t = 0; t < nt; t++) memcpy(xsub + (size_t)t * D, x + (size_t)tl[t] * D, (size_t)D * 4);
            oracle_matmul_q4r4_s(g, xsub, ex->g + (size_t)e * gq, ex->gs + (size_t)e * gsn, nt, D, I);
            oracle_matmul_q4r4_s(u, xsub, ex->u + (size_t)e * gq, ex->us + (size_t)e * gsn, nt, D, I);
            oracle_silu_mul(g, u, (int64_t)nt * I);
            oracle_matmul_q4r4_s(h, g, ex->d + (size_t)e * dq, ex->ds + (size_t)e * dsn, nt, I, D);
            for (int t = 0; t < nt; t++)
                for (int k = 0; k < K; k++)
                    if (idx[(size_t)tl[t] * K + k] == e) {
                        float wk = rw[(size_t)tl[t] * K + k];
                        float *o = out + (size_t)tl[t] * D;
                        for (int dd = 0; dd < D; dd++) o[dd] = fmaf(wk, h[(size_t)t * D + dd], o[dd]);
                    }
        }
    }
    if (idx_out) memcpy(idx_out, idx, sizeof(int) * (size_t)S * K);
    if (w_out) memcpy(w_out, rw, sizeof(float) * (size_t)S * K);
    free(idx); free(rw); free(tl); free(xsub); free(g); free(u); free(h);
}

/* ------------------------------------------------------------------ */
/* Attention core between the projections (nn/attn.c:29-74)            */
/* ------------------------------------------------------------------ */

/* hw/hw_ops.h:14-18 -- RMS norm of one head: mean of squares in double, then x * r * w. */
static void attn_rmsnorm(float *out, const float *x, const float *w, int n, float eps) {
    double ms = 0;
    for (int i = 0; i < n; i++) ms += (double)x[i] * x[i];
    float r = 1.f / sqrtf((float)(ms / n) + eps);
    for (int i = 0; i < n; i++) out[i] = x[i] * r * w[i];
}

/* nn/rope.c:39-49 -- half-split rotation of the first rot dimensions of a head;
 * angle = pos / powf(theta, 2i / rot) (the cached table holds the same expression). */
ORACLE_API void oracle_rope_head(float *x, int pos, float theta, int rot) {
    for (int i = 0; i < rot / 2; i++) {
        float angle = pos / powf(theta, (float)(2 * i) / rot);
        float c = cosf(angle), s = sinf(angle);
        float a = x[i], b = x[i + rot / 2];
        x[i] = a * c - b * s;
        x[i + rot / 2] = a * s + b * c;
    }
}

/* nn/attn.c:29-74 (attn_tail without the projections and the optional gate): q [S][H*hd], k, v
 * [S][KV*hd] are the projected rows of tokens pos_base .. pos_base+S-1.  QK-norm (qn/kn per head
 * dimension, NULL = none) and RoPE in place; K and V rows go to the cache at their positions --
 * f32 (K, V: [KV][max_t][hd]) or, when K8 is given, int8 rows with one scale per (head, position)
 * from qrow_i8 (nn/mat.c:15-17); per (head, token): scores against positions 0..pos
 * (hw/hw_ops.h:53-55, hw/hw_scalar.h:24-34; int8 keys: Ks * dot * scale, nn/attn_kernels.c:14-17),
 * softmax (hw/hw_ops.h:22-26), accumulation over positions in order (hw/hw_ops.h:56-59; int8 values:
 * nn/attn_kernels.c:26-35).  ctx [S][H*hd].  Plain f32 statements, nothing contracted: the
 * reference's tiers differ in summation order here, parity is by tolerance. */
/* engines/gemma.c:287-297 -- p-RoPE: pairs (j, j + hd/2), rotated for j < rot_angles, frequency theta^(-2j/hd),
 * angle = pos * that. */
ORACLE_API void oracle_gemma_rope_head(float *x, int pos, float theta, int hd, int rot_angles) {
    int h = hd / 2;
    for (int j = 0; j < rot_angles && j < h; j++) {
        float inv = powf(theta, -2.0f * j / hd);
        float ang = pos * inv, cs = cosf(ang), sn = sinf(ang);
        float a = x[j], b = x[j + h];
        x[j] = a * cs - b * sn;
        x[j + h] = b * cs + a * sn;
    }
}

static void attn_core_impl(float *ctx, float *q, float *k, float *v, int S, int pos_base,
                           int H, int KV, int hd, float theta, float eps, int rot,
                           const float *qn, const float *kn,
                           float *K, float *V, int8_t *K8, int8_t *V8, float *Ks, float *Vs, int max_t,
                           int gemma, int window, float scale_in, const float *vn);
ORACLE_API void oracle_attn_core(float *ctx, float *q, float *k, const float *v, int S, int pos_base,
                                 int H, int KV, int hd, float theta, float eps, int rot,
                                 const float *qn, const float *kn,
                                 float *K, float *V, int8_t *K8, int8_t *V8, float *Ks, float *Vs, int max_t) {
    attn_core_impl(ctx, q, k, (float *)v, S, pos_base, H, KV, hd, theta, eps, rot, qn, kn, K, V, K8, V8, Ks, Vs, max_t, 0, 0, 0.f, NULL);
}
/* engines/gemma.c:299-386 (attention() without the projections, shared-KV layers and k_eq_v): the same steps with
 * gemma's own pieces -- norm gains given as the multipliers (1 + w with the default zc_norm, :279-284), an optional
 * VALUE norm (vn, :320-324; v is normed in place), p-RoPE (rot = rotated pairs; hd/2 on sliding layers, :306), score
 * scale 1/sqrt(query_pre_attn_scalar) when given (:363), and on sliding layers only positions
 * max(0, qpos - window + 1) .. qpos (:373).  window = 0: a global layer. */
ORACLE_API void oracle_attn_core_gemma(float *ctx, float *q, float *k, float *v, int S, int pos_base,
                                       int H, int KV, int hd, float theta, float eps, int rot_angles,
                                       const float *qn, const float *kn, const float *vn, int window, float scale,
                                       float *K, float *V, int8_t *K8, int8_t *V8, float *Ks, float *Vs, int max_t) {
    attn_core_impl(ctx, q, k, v, S, pos_base, H, KV, hd, theta, eps, rot_angles, qn, kn, K, V, K8, V8, Ks, Vs, max_t, 1, window, scale, vn);
}
static void attn_core_impl(float *ctx, float *q, float *k, float *v, int S, int pos_base,
                           int H, int KV, int hd, float theta, float eps, int rot,
                           const float *qn, const float *kn,
                           float *K, float *V, int8_t *K8, int8_t *V8, float *Ks, float *Vs, int max_t,
                           int gemma, int window, float scale_in, const float *vn) {
    int G = H / KV;
    size_t qw = (size_t)H * hd, kw = (size_t)KV * hd;
    for (int s = 0; s < S; s++) {
        int pos = pos_base + s;
        for (int hh = 0; hh < H; hh++) {
            float *p = q + s * qw + (size_t)hh * hd;
            if (qn) attn_rmsnorm(p, p, qn, hd, eps);
            if (gemma) oracle_gemma_rope_head(p, pos, theta, hd, rot); else oracle_rope_head(p, pos, theta, rot);
        }
        for (int hh = 0; hh < KV; hh++) {
            float *p = k + s * kw + (size_t)hh * hd;
            if (kn) attn_rmsnorm(p, p, kn, hd, eps);
            if (gemma) oracle_gemma_rope_head(p, pos, theta, hd, rot); else oracle_rope_head(p, pos, theta, rot);
            if (vn) { float *pv = v + s * kw + (size_t)hh * hd; attn_rmsnorm(pv, pv, vn, hd, eps); }
        }
    }
    for (int s = 0; s < S; s++)
        for (int hh = 0; hh < KV; hh++) {
            size_t slot = (size_t)hh * max_t + pos_base + s;
            if (K8) {
                Ks[slot] = oracle_qrow_i8(k + s * kw + (size_t)hh * hd, K8 + slot * hd, hd);
                Vs[slot] = oracle_qrow_i8(v + s * kw + (size_t)hh * hd, V8 + slot * hd, hd);
            } else {
                memcpy(K + slot * hd, k + s * kw + (size_t)hh * hd, sizeof(float) * hd);
                memcpy(V + slot * hd, v + s * kw + (size_t)hh * hd, sizeof(float) * hd);
            }
        }
    float scale = scale_in > 0.f ? scale_in : 1.f / sqrtf((float)hd);
    #pragma omp parallel
    {
        float *sc = (float *)malloc(sizeof(float) * (size_t)(pos_base + S + 1));
        #pragma omp for schedule(static)
        for (int r = 0; r < H * S; r++) {
            int hh = r / S, s = r % S, kvh = hh / G, qpos = pos_base + s;
            int t0 = window > 0 && qpos - window + 1 > 0 ? qpos - window + 1 : 0;
            int n = qpos + 1 - t0;
            const float *qv = q + s * qw + (size_t)hh * hd;
            size_t base = (size_t)kvh * max_t + t0;                     /* positions t0 .. qpos, indexed from 0 below */
            for (int t = 0; t < n; t++) {
                float d = 0.f;
                if (K8) {
                    const int8_t *kr = K8 + (base + t) * hd;
                    for (int i = 0; i < hd; i++) d += qv[i] * (float)kr[i];
                    sc[t] = Ks[base + t] * d * scale;
                } else {
                    const float *kr = K + (base + t) * hd;
                    for (int i = 0; i < hd; i++) d += qv[i] * kr[i];
                    sc[t] = d * scale;
                }
            }
            float m = -1e30f, sum = 0.f;
            for (int t = 0; t < n; t++) if (sc[t] > m) m = sc[t];
            for (int t = 0; t < n; t++) { sc[t] = oracle_expf(sc[t] - m); sum += sc[t]; }
            for (int t = 0; t < n; t++) sc[t] /= sum;
            float *cx = ctx + s * qw + (size_t)hh * hd;
            for (int i = 0; i < hd; i++) cx[i] = 0.f;
            for (int t = 0; t < n; t++) {
                if (V8) {
                    const int8_t *vr = V8 + (base + t) * hd;
                    float a = sc[t] * Vs[base + t];
                    for (int i = 0; i < hd; i++) cx[i] += a * (float)vr[i];
                } else {
                    const float *vr = V + (base + t) * hd;
                    for (int i = 0; i < hd; i++) cx[i] += sc[t] * vr[i];
                }
            }
        }
        free(sc);
    }
}
