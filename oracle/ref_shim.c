/* ref_shim.c -- glue compiled TOGETHER WITH the unmodified reference sources
 * into oracle/_ref/libmoty_ref*.so (see oracle/Makefile).  TEST INFRASTRUCTURE
 * ONLY: it lets the test-suite and the benchmark's CPU arm call reference
 * functions that are static or need reference structs built around plain
 * arrays.  It contains no arithmetic of its own: every number comes out of a
 * reference function.
 *
 * Reference entry points used (moty source tree, directory c/):
 *   moty_nn_moe_topk_d1 / _batch, moty_nn_moe_sigmoid_d1 / _batch   nn/moe.c:154-156, 207-208
 *   moty_expert_cache_init/get     runtime/moecache.c:4-18, 50-89
 *   moty_matmul_q, moty_softmax_row, moty_moe_topk   (OLMoE block, engines/olmoe.c:219-244)
 *   moty_pack_q4r4_block           nn/quant.c:157-179
 *   moty_mat_apply                 nn/mat.c:70-83
 */
#include "nn/moe.h"
#include "nn/ffn.h"
#include "nn/nn_matmul.h"
#include "nn/nn_norm.h"
#include "nn/nn_quant.h"
#include "nn/par.h"
#include <string.h>

typedef struct {
    int E, K, I, D;
    const int8_t *g, *u, *d;       /* [E][I][D], [E][I][D], [E][D][I] */
    const float *gs, *us, *ds;     /* [E][I], [E][I], [E][D] */
} ShimExperts;

/* LoadExpertFn: copy one expert out of the caller's expert-major arrays */
static void shim_load_expert(void *ctx, int layer, int eid, ExpertSlot *s, int inter, int hidden) {
    const ShimExperts *ex = ctx; (void)layer;
    size_t n = (size_t)inter * hidden;
    memcpy(s->g, ex->g + (size_t)eid * n, n);
    memcpy(s->u, ex->u + (size_t)eid * n, n);
    memcpy(s->d, ex->d + (size_t)eid * n, n);
    memcpy(s->gs, ex->gs + (size_t)eid * inter, sizeof(float) * inter);
    memcpy(s->us, ex->us + (size_t)eid * inter, sizeof(float) * inter);
    memcpy(s->ds, ex->ds + (size_t)eid * hidden, sizeof(float) * hidden);
}

/* the same for experts stored as per-row int4 (ebits <= 4: nibble rows, element 2j in the low nibble; nn/moe.h:12):
 * ex->g / u / d then point at [E][I][(D+1)/2], [E][I][(D+1)/2], [E][D][(I+1)/2] bytes */
static void shim_load_expert_i4(void *ctx, int layer, int eid, ExpertSlot *s, int inter, int hidden) {
    const ShimExperts *ex = ctx; (void)layer;
    size_t ngu = (size_t)inter * ((hidden + 1) / 2), nd = (size_t)hidden * ((inter + 1) / 2);
    memcpy(s->g, ex->g + (size_t)eid * ngu, ngu);
    memcpy(s->u, ex->u + (size_t)eid * ngu, ngu);
    memcpy(s->d, ex->d + (size_t)eid * nd, nd);
    memcpy(s->gs, ex->gs + (size_t)eid * inter, sizeof(float) * inter);
    memcpy(s->us, ex->us + (size_t)eid * inter, sizeof(float) * inter);
    memcpy(s->ds, ex->ds + (size_t)eid * hidden, sizeof(float) * hidden);
}

/* The reference MoE block with a softmax/top-k gate, all experts resident
 * (cache capacity = E, so nothing is ever evicted), no shared expert.
 * router_fmt: WF_F32 (router_f = [E][D] floats) or WF_I8 (router_q + router_qs).
 * S == 1 takes the decode path, S > 1 the batch path. */
static void shim_moe_block(const ShimExperts *ex, int router_fmt, const float *router_f, const int8_t *router_q,
                           const float *router_qs, const float *x, int S, float *out, int sig, const float *bias, int ebits);
/* either gate over per-row int4 experts (the decode path is integer throughout; the batch path goes through
 * moty_matmul_i4_s, whose integer form needs IDOT4=1 in the environment before its first call) */
void refshim_moe_i4(const ShimExperts *ex, int router_fmt, const float *router_f, const int8_t *router_q,
                    const float *router_qs, int sig, const float *bias, const float *x, int S, float *out) {
    shim_moe_block(ex, router_fmt, router_f, router_q, router_qs, x, S, out, sig, bias, 4);
}
void refshim_moe_topk(const ShimExperts *ex, int router_fmt, const float *router_f,
                      const int8_t *router_q, const float *router_qs,
                      const float *x, int S, float *out) {
    shim_moe_block(ex, router_fmt, router_f, router_q, router_qs, x, S, out, 0, NULL, 8);
}
/* the same block behind the sigmoid + expert-bias gate of LFM2 (moty_nn_moe_sigmoid_d1 / _batch, nn/moe.c:154,207) */
void refshim_moe_sigmoid(const ShimExperts *ex, int router_fmt, const float *router_f,
                         const int8_t *router_q, const float *router_qs, const float *bias,
                         const float *x, int S, float *out) {
    shim_moe_block(ex, router_fmt, router_f, router_q, router_qs, x, S, out, 1, bias, 8);
}
static void shim_moe_block(const ShimExperts *ex, int router_fmt, const float *router_f, const int8_t *router_q,
                           const float *router_qs, const float *x, int S, float *out, int sig, const float *bias, int ebits) {
    Mat router; mat_reset_storage(&router);
    router.fmt = router_fmt; router.O = ex->E; router.I = ex->D;
    router.f = (float *)router_f; router.q = (int8_t *)router_q; router.qs = (float *)router_qs;
    ExpertCache ec; moty_expert_cache_init(&ec, ex->E, ex->E);
    Scratch scr; memset(&scr, 0, sizeof scr);
    MotyMoeView v; memset(&v, 0, sizeof v);
    v.router = &router; v.ec = &ec; v.load_expert = ebits <= 4 ? shim_load_expert_i4 : shim_load_expert; v.ectx = (void *)ex;
    v.E = ex->E; v.K = ex->K; v.I = ex->I; v.D = ex->D; v.li = 0; v.ebits = ebits; v.scr = &scr;
    v.expert_bias = bias;
    if (sig) { if (S == 1) moty_nn_moe_sigmoid_d1(&v, x, out); else moty_nn_moe_sigmoid_batch(&v, x, S, out); }
    else if (S == 1) moty_nn_moe_topk_d1(&v, x, out);
    else moty_nn_moe_topk_batch(&v, x, S, out);
    moty_expert_cache_free(&ec);
    moty_scr_free(&scr);
}

/* engines/olmoe.c:219-244 is a static function of an engine translation unit;
 * this is the same sequence of reference calls on caller-provided logits
 * (the f32 router matmul that produces them sits outside the quantized path). */
void refshim_olmoe_moe(const ShimExperts *ex, const float *x, int S, float *logits, float *out,
                       int norm_topk, int *idx_out, float *w_out) {
    int E = ex->E, K = ex->K, I = ex->I, D = ex->D;
    float *g = moty_falloc(I), *u = moty_falloc(I), *hh = moty_falloc(D);
    memset(out, 0, (size_t)S * D * sizeof(float));
    for (int s = 0; s < S; s++) {
        int idx[64]; float w[64];
        float *pr = logits + (size_t)s * E;
        moty_softmax_row(pr, E);
        moty_moe_topk(pr, E, K, idx, w, norm_topk);
        const float *xs = x + (size_t)s * D;
        for (int kk = 0; kk < K; kk++) {
            size_t e = (size_t)idx[kk];
            moty_matmul_q(g, xs, ex->g + e * I * D, ex->gs + e * I, D, I);
            moty_matmul_q(u, xs, ex->u + e * I * D, ex->us + e * I, D, I);
            moty_hw_silu_mul_ref(g, u, I);
            moty_matmul_q(hh, g, ex->d + e * D * I, ex->ds + e * D, I, D);
            float weight = w[kk];
            float *os = out + (size_t)s * D;
            for (int d = 0; d < D; d++) os[d] += weight * hh[d];
        }
        if (idx_out) memcpy(idx_out + (size_t)s * K, idx, sizeof(int) * K);
        if (w_out) memcpy(w_out + (size_t)s * K, w, sizeof(float) * K);
    }
    free(g); free(u); free(hh);
}

/* softmax + top-k exactly as the static route_topk of nn/moe.c:27-30 */
void refshim_route_topk(float *logits, int E, int K, int *idx, float *w) {
    moty_softmax_row(logits, E);
    moty_moe_topk(logits, E, K, idx, w, 1);
}

/* a whole matrix through moty_pack_q4r4_block, 4 rows at a time
 * (what runtime/rt_model_load.h r4_pack_part does at load) */
void refshim_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16) {
    int nb = I / 32;
    for (int b = 0; b < (O + 3) / 4; b++) {
        int nr = O - 4 * b < 4 ? O - 4 * b : 4;
        moty_pack_q4r4_block(w + (size_t)b * 4 * I, nr, I, q4 + (size_t)b * nb * 64, s16 + (size_t)b * nb * 4);
    }
}

/* the same for Q8R4 (moty_pack_q8r4_block, nn/quant.c:135-155) */
void refshim_pack_q8r4(const float *w, int O, int I, int8_t *q8, uint16_t *s16) {
    int nb = I / 32;
    for (int b = 0; b < (O + 3) / 4; b++) {
        int nr = O - 4 * b < 4 ? O - 4 * b : 4;
        moty_pack_q8r4_block(w + (size_t)b * 4 * I, nr, I, q8 + (size_t)b * nb * 128, s16 + (size_t)b * nb * 4);
    }
}

/* moty_nn_dense_ffn (nn/ffn.c:26-55) over three WF_I8 or three WF_Q4R4 matrices */
void refshim_dense_ffn(int fmt, const void *gq, const void *gs, const void *uq, const void *us,
                       const void *dq, const void *ds, int D, int I, const float *x, int S, float *out) {
    Mat g, u, d; mat_reset_storage(&g); mat_reset_storage(&u); mat_reset_storage(&d);
    g.fmt = u.fmt = d.fmt = fmt;
    g.O = I; g.I = D; u.O = I; u.I = D; d.O = D; d.I = I;
    if (fmt == WF_I8) {
        g.q = (int8_t *)gq; g.qs = (float *)gs; u.q = (int8_t *)uq; u.qs = (float *)us;
        d.q = (int8_t *)dq; d.qs = (float *)ds;
    } else {
        g.q4 = (uint8_t *)gq; g.s16 = (uint16_t *)gs; u.q4 = (uint8_t *)uq; u.s16 = (uint16_t *)us;
        d.q4 = (uint8_t *)dq; d.s16 = (uint16_t *)ds;
    }
    Scratch scr; memset(&scr, 0, sizeof scr);
    MotyFfnView f = { .gate = &g, .up = &u, .down = &d, .gate_up = NULL, .inter = I, .scr = &scr };
    moty_nn_dense_ffn(&f, x, S, out);
    moty_scr_free(&scr);
}

void refshim_set_threads(int n) { moty_par_set_threads(n); }
int  refshim_threads(void) { return moty_par_threads(); }
