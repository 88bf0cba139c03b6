/* qwen_cuda.c -- the reference's `qwen` engine, source untouched, with the CUDA backend attached.
 *
 * The engine is pulled in as one translation unit, the way the reference's own tests do
 * (tests/qwen_tests.c:4-5), so this file sees its static loader and step().  main() below is
 * engine_main (runtime/runtime.h:117-180) reduced to the REF= validation route, plus the two calls
 * a maintainer adds to the loader: moty_hw_cuda_open() and one moty_hw_cuda_attach() per loaded
 * matrix.  Nothing else differs: tokens, attention, norms, sampling and the loop are the reference's.
 *
 *   SNAP=<dir> QBITS=8 REF=<ref.json> MOTY_CUDA=1 ./qwen_cuda      the matmuls run on GPU 0
 *   SNAP=<dir> QBITS=8 REF=<ref.json> MOTY_CUDA=0 ./qwen_cuda      the reference as it is (CPU)
 *   SNAP=<dir> QBITS=8 REF=<ref.json> MOTY_CUDA=2 ./qwen_cuda      the whole step() on GPU 0: activations stay on the device
 *                                                                 between the library's *_dev entries (see shim_step_dev)
 *   MOTY_GPU=<ordinal>                                            another GPU
 *   MOTY_SHIM_TRACE=<file>  instead of run_ref's summary: the same greedy loop (runtime/rt_gen_loop.h:46-84)
 *       with prefill and decode timed apart and one line per generated token written to <file>:
 *       "<step> <token id> <top-1 logit bits> <top-2 logit bits> <FNV-1a hash of the whole logit row>",
 *       so that two runs can be compared logit row by logit row without storing 152 k floats per step.
 *   MOTY_SHIM_FORCE=1  (with MOTY_SHIM_TRACE) teacher forcing: the token fed to the next step is the REF file's
 *       full_ids entry, not the run's own pick (which is still recorded), so that two runs whose arithmetic differs in
 *       the last bits can be compared step by step on identical contexts.
 */
#define QWEN_TEST                     /* engines/qwen.c:780: no main() from the engine */
#include "engines/qwen.c"
#include "hw_cuda.h"
#include "moty_cuda.h"

static int shim_attach_model(Model *m, int dev) {
    int n = 0;
    for (int i = 0; i < m->c.n_layers && i < m->base.n_resident; i++) {
        Layer *l = &m->L[i];
        /* fused [q|k|v] and [gate|up] views replace their sources where qwen_fuse built them (engines/qwen.c:389-396) */
        if (l->qkv.q4) n += moty_hw_cuda_attach(&l->qkv, dev);
        else { n += moty_hw_cuda_attach(&l->q, dev); n += moty_hw_cuda_attach(&l->k, dev); n += moty_hw_cuda_attach(&l->v, dev); }
        n += moty_hw_cuda_attach(&l->o, dev);
        if (l->gate_up.q4) n += moty_hw_cuda_attach(&l->gate_up, dev);
        else { n += moty_hw_cuda_attach(&l->gate, dev); n += moty_hw_cuda_attach(&l->up, dev); }
        n += moty_hw_cuda_attach(&l->down, dev);
        Mat *lin[5] = { &l->aqkv, &l->az, &l->ab, &l->aa, &l->aout };
        for (int j = 0; j < 5; j++) n += moty_hw_cuda_attach(lin[j], dev);
    }
    n += moty_hw_cuda_attach(&m->base.lm_head, dev);      /* tied: the int8 embedding table (rt_model_load.h:459-460) */
    return n;
}

/* ---- MOTY_CUDA=2: step() (engines/qwen.c:681-740) with the activations resident on the GPU ------------------------
 * The same sequence of operations, each one a *_dev entry of the C ABI on the library's stream: embed_row ->
 * per layer { rmsnorm, q/k/v products, attention core (QK-norm, RoPE, KV store, scores: the layer's KV cache lives in
 * its MotyCudaAttn), o product, residual add + norm, dense FFN, residual add } -> final norm of the last row ->
 * lm_head.  One copy in (the token ids) and one copy out (the logits row) per step.  For dense layers with int8
 * matrices, a tied int8 head and f32 or int8 KV (what QBITS=8 gives); anything else is refused.  The matmuls and
 * quantizers are bit-exact; the attention core sums in another order than the CPU tier (a few 1e-6), so the logits
 * agree to that and the greedy ids are compared, not the hashes. */
typedef struct {
    int dev, cap_S, max_t;
    float *x, *nrm, *tmp, *q, *k, *v, *ctx, *logits, *final_norm;
    float *hlogits;                   /* page-locked: the logits row of the latest step (returned to the loop, never freed by it) */
    int *ids, *pos;                   /* token ids of the step; the first position, for the captured decode step */
    float **in_ln, **post_ln;
    MotyCudaAttn **attn;
    MotyCudaGraph *graph;             /* one decode token, captured after the first one has run (MOTY_SHIM_GRAPH=0: never) */
    int decoded;
} ShimDev;
static ShimDev g_sd;

#define SHIM_CK(call) do { if ((call) != 0) moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] %s: %s\n", #call, moty_cuda_last_error()); } while (0)

static float *shim_dev_f32(const float *host, int64_t n, int dev) {
    void *p = NULL;
    SHIM_CK(moty_cuda_dev_alloc(&p, (size_t)n * 4, dev));
    if (host) SHIM_CK(moty_cuda_dev_upload(p, host, (size_t)n * 4, dev, NULL));
    return p;
}

static void shim_dev_init(Model *m, int dev, int cap_S, int max_t) {
    Cfg *c = &m->c; ShimDev *d = &g_sd;
    int D = c->hidden, H = c->n_heads, KV = c->n_kv_heads, hd = c->head_dim;
    if (!m->base.lm_tied || m->base.lm_head.fmt != WF_I8 || !m->base.lm_head.sh)
        moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] MOTY_CUDA=2 wants the tied int8 head on the GPU (QBITS=8)\n");
    d->dev = dev; d->cap_S = cap_S; d->max_t = max_t;
    d->x = shim_dev_f32(NULL, (int64_t)cap_S * D, dev); d->nrm = shim_dev_f32(NULL, (int64_t)cap_S * D, dev);
    d->tmp = shim_dev_f32(NULL, (int64_t)cap_S * D, dev);
    d->q = shim_dev_f32(NULL, (int64_t)cap_S * H * hd, dev); d->ctx = shim_dev_f32(NULL, (int64_t)cap_S * H * hd, dev);
    d->k = shim_dev_f32(NULL, (int64_t)cap_S * KV * hd, dev); d->v = shim_dev_f32(NULL, (int64_t)cap_S * KV * hd, dev);
    d->logits = shim_dev_f32(NULL, c->vocab, dev);
    d->final_norm = shim_dev_f32(m->base.final_norm, D, dev);
    /* ids[0] and the position sit side by side: a decode token uploads both with one copy (a prompt needs no position
     * on the device and may use the whole buffer) */
    void *ids = NULL; SHIM_CK(moty_cuda_dev_alloc(&ids, ((size_t)cap_S + 1) * 4, dev)); d->ids = ids;
    d->pos = d->ids + 1;
    void *hl = NULL; SHIM_CK(moty_cuda_host_alloc(&hl, (size_t)c->vocab * 4)); d->hlogits = hl;
    d->graph = NULL; d->decoded = 0;
    d->in_ln = calloc(c->n_layers, sizeof(float *)); d->post_ln = calloc(c->n_layers, sizeof(float *));
    d->attn = calloc(c->n_layers, sizeof(MotyCudaAttn *));
    for (int i = 0; i < c->n_layers; i++) {
        Layer *l = &m->L[i];
        if (l->type != LT_FULL || l->gated || l->lo || !l->q.sh || !l->k.sh || !l->v.sh || !l->o.sh || !l->gate.sh || !l->up.sh || !l->down.sh)
            moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] MOTY_CUDA=2: layer %d is not a plain dense attention layer with its matrices on the GPU\n", i);
        d->in_ln[i] = shim_dev_f32(l->in_ln, D, dev); d->post_ln[i] = shim_dev_f32(l->post_ln, D, dev);
        SHIM_CK(moty_cuda_attn_create(&d->attn[i], H, KV, hd, c->rot, c->theta, c->eps, l->qn, l->kn, max_t, g_kv_bits == 8, dev));
    }
    SHIM_CK(moty_cuda_sync(dev));
}

/* MOTY_SHIM_CHECK=1: on the first step, layer 0's stages are also computed by the reference's own functions on the host
 * (embed_row, rmsnorm_row, attention(), mlp(): the matmuls inside go through the hook and are bit-exact) and the largest
 * difference to the device buffers is printed per stage -- a wiring check for whoever changes the step. */
static void shim_check(const char *what, const float *dev_buf, const float *host, int64_t n, int dev) {
    float *tmp = falloc(n);
    SHIM_CK(moty_cuda_dev_download(tmp, dev_buf, (size_t)n * 4, dev, NULL));
    double worst = 0, mag = 0;
    for (int64_t i = 0; i < n; i++) { double e = fabs((double)tmp[i] - host[i]); if (e > worst) worst = e; if (fabs(host[i]) > mag) mag = fabs(host[i]); }
    fprintf(stderr, "[check] %-28s max |diff| %.3g of magnitude %.3g\n", what, worst, mag);
    free(tmp);
}

/* the operations of one step on the device buffers; pos_dev != NULL: one token whose position is read from the device
 * (the form a captured graph can replay).  A residual add and the norm after it are one launch, as in the reference's
 * fused add+norm (hw/hw_ops.h:30-32 then :14-18; same bits). */
static void shim_layers(Model *m, int S, int pos_base, const int *pos_dev, int check, const int *ids) {
    Cfg *c = &m->c; ShimDev *d = &g_sd;
    int D = c->hidden;
    float *hx = NULL, *hn = NULL, *ht = NULL;
    SHIM_CK(moty_cuda_embed_rows_dev((MotyCudaMat *)m->base.lm_head.sh, d->x, d->ids, S, 1.f, NULL));
    if (check) {
        kv_alloc(m, d->max_t);
        hx = falloc((int64_t)S * D); hn = falloc((int64_t)S * D); ht = falloc((int64_t)S * D);
        for (int s = 0; s < S; s++) embed_row(m, ids[s], 1.f, hx + (int64_t)s * D);
        shim_check("embed", d->x, hx, (int64_t)S * D, d->dev);
    }
    SHIM_CK(moty_cuda_rmsnorm_dev(d->nrm, d->x, d->in_ln[0], S, D, c->eps, NULL));
    for (int i = 0; i < c->n_layers; i++) {
        Layer *l = &m->L[i];
        if (check && i == 0) {
            for (int s = 0; s < S; s++) rmsnorm_row(hn + (int64_t)s * D, hx + (int64_t)s * D, l->in_ln, D, c->eps);
            shim_check("layer 0 input norm", d->nrm, hn, (int64_t)S * D, d->dev);
            attention(m, l, 0, hn, S, pos_base, ht);
        }
        if (S == 1 && l->q.I <= 4096) {                 /* a decode token: the three projections share their row -> one launch */
            MotyCudaMat *w3[3] = { (MotyCudaMat *)l->q.sh, (MotyCudaMat *)l->k.sh, (MotyCudaMat *)l->v.sh };
            float *y3[3] = { d->q, d->k, d->v };
            const float *x3[3] = { d->nrm, d->nrm, d->nrm };
            SHIM_CK(moty_cuda_mat_apply_multi_dev(3, w3, y3, x3, NULL));
        } else {
            SHIM_CK(moty_cuda_mat_apply_dev((MotyCudaMat *)l->q.sh, d->q, d->nrm, S, NULL));
            SHIM_CK(moty_cuda_mat_apply_dev((MotyCudaMat *)l->k.sh, d->k, d->nrm, S, NULL));
            SHIM_CK(moty_cuda_mat_apply_dev((MotyCudaMat *)l->v.sh, d->v, d->nrm, S, NULL));
        }
        if (pos_dev) SHIM_CK(moty_cuda_attn_core_posdev(d->attn[i], d->ctx, d->q, d->k, d->v, S, pos_dev, d->max_t - 1, NULL));
        else SHIM_CK(moty_cuda_attn_core_dev(d->attn[i], d->ctx, d->q, d->k, d->v, S, pos_base, NULL));
        SHIM_CK(moty_cuda_mat_apply_dev((MotyCudaMat *)l->o.sh, d->tmp, d->ctx, S, NULL));
        if (check && i == 0) shim_check("layer 0 attention + o", d->tmp, ht, (int64_t)S * D, d->dev);
        SHIM_CK(moty_cuda_add_rmsnorm_dev(d->x, d->tmp, d->nrm, d->post_ln[i], S, D, c->eps, NULL));      /* x += attn; nrm = norm(x) */
        if (check && i == 0) {
            moty_hw_add(hx, ht, (int64_t)S * D);
            for (int s = 0; s < S; s++) rmsnorm_row(hn + (int64_t)s * D, hx + (int64_t)s * D, l->post_ln, D, c->eps);
            shim_check("layer 0 residual", d->x, hx, (int64_t)S * D, d->dev);
            shim_check("layer 0 post-attention norm", d->nrm, hn, (int64_t)S * D, d->dev);
            mlp(m, l, hn, S, ht);
        }
        SHIM_CK(moty_cuda_ffn_dev((MotyCudaMat *)l->gate.sh, (MotyCudaMat *)l->up.sh, (MotyCudaMat *)l->down.sh, MOTY_ACT_SILU,
                                  d->tmp, d->nrm, S, NULL));
        if (check && i == 0) { shim_check("layer 0 FFN", d->tmp, ht, (int64_t)S * D, d->dev); free(hx); free(hn); free(ht); }
        if (i + 1 < c->n_layers)                        /* x += ffn; nrm = the next layer's input norm */
            SHIM_CK(moty_cuda_add_rmsnorm_dev(d->x, d->tmp, d->nrm, d->in_ln[i + 1], S, D, c->eps, NULL));
        else
            SHIM_CK(moty_cuda_add_dev(d->x, d->tmp, (long long)S * D, NULL));
    }
    SHIM_CK(moty_cuda_rmsnorm_dev(d->nrm, d->x + (int64_t)(S - 1) * D, d->final_norm, 1, D, c->eps, NULL));
    SHIM_CK(moty_cuda_mat_apply_dev((MotyCudaMat *)m->base.lm_head.sh, d->logits, d->nrm, 1, NULL));
}

/* returns the logits of the last token (malloc'd), like step().  Decode tokens after the first are replayed from a
 * CUDA graph of one token (captured through the library, which holds the stream): the token id and the position are
 * uploaded in front of each replay. */
static float *shim_step_dev(Model *m, const int *ids, int S, int pos_base) {
    Cfg *c = &m->c; ShimDev *d = &g_sd;
    if (S > d->cap_S || pos_base + S > d->max_t) moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] step of %d tokens at %d exceeds the device buffers\n", S, pos_base);
    static int checked;
    const int check = !checked && getenv("MOTY_SHIM_CHECK") && atoi(getenv("MOTY_SHIM_CHECK"));
    checked = 1;
    static int use_graph = -1;
    if (use_graph < 0) { const char *e = getenv("MOTY_SHIM_GRAPH"); use_graph = e ? atoi(e) : 1; }
    if (S == 1 && use_graph && !check) {
        const int idpos[2] = { ids[0], pos_base };
        SHIM_CK(moty_cuda_dev_upload(d->ids, idpos, 8, d->dev, NULL));
        if (!d->graph && d->decoded >= 1) {             /* the token before this one ran the same sequence uncaptured */
            SHIM_CK(moty_cuda_graph_begin(d->dev, NULL));
            shim_layers(m, 1, pos_base, d->pos, 0, ids);
            SHIM_CK(moty_cuda_graph_end(&d->graph, d->dev, NULL));
        }
        if (d->graph) SHIM_CK(moty_cuda_graph_launch(d->graph));
        else shim_layers(m, 1, pos_base, d->pos, 0, ids);
        d->decoded++;
    } else {
        SHIM_CK(moty_cuda_dev_upload(d->ids, ids, (size_t)S * 4, d->dev, NULL));
        shim_layers(m, S, pos_base, NULL, check, ids);
    }
    m->base.kv_len = pos_base + S;
    SHIM_CK(moty_cuda_dev_download(d->hlogits, d->logits, (size_t)c->vocab * 4, d->dev, NULL));
    SHIM_CK(moty_cuda_kernel_status(d->dev, NULL));
    return d->hlogits;
}

static int g_shim_resident;
static float *shim_step_any(Model *m, const int *ids, int S, int pos_base) {
    return g_shim_resident ? shim_step_dev(m, ids, S, pos_base) : step(m, ids, S, pos_base);
}

/* FNV-1a over 64-bit words (the row is a multiple of 4 bytes; a last half word is taken alone): the trace hashes 600 KB
 * per token, and byte by byte that cost more than the GPU's whole step */
static uint64_t shim_fnv(const void *p, size_t n) {
    const unsigned char *b = p; uint64_t h = 1469598103934665603ULL;
    size_t i = 0;
    for (; i + 8 <= n; i += 8) { uint64_t w; memcpy(&w, b + i, 8); h ^= w; h *= 1099511628211ULL; }
    for (; i < n; i++) { h ^= b[i]; h *= 1099511628211ULL; }
    return h;
}

static void shim_trace_row(FILE *f, int step_no, const float *logit, int V, int best) {
    float top2 = -INFINITY;
    for (int i = 0; i < V; i++) if (i != best && logit[i] > top2) top2 = logit[i];
    uint32_t b1, b2; memcpy(&b1, &logit[best], 4); memcpy(&b2, &top2, 4);
    fprintf(f, "%d %d %08x %08x %016llx\n", step_no, best, b1, b2, (unsigned long long)shim_fnv(logit, (size_t)V * 4));
}

/* run_ref's loop (runtime/rt_gen_loop.h:46-84) with the two phases timed apart and a trace */
static int shim_run_trace(Model *m, const char *refpath, const char *tracepath) {
    char *buf = slurp_file(refpath, NULL);
    jval *ref = json_parse(buf);
    int np, nfull;
    int *prompt = read_int_array(ref, "prompt_ids", &np);
    int *full = read_int_array(ref, "full_ids", &nfull);
    int n_new = nfull - np;
    if (n_new <= 0) { fprintf(stderr, "ref.json: full_ids does not extend prompt_ids\n"); return 1; }
    FILE *tf = fopen(tracepath, "w");
    if (!tf) { perror(tracepath); return 1; }
    if (g_shim_resident) shim_dev_init(m, g_sd.dev, np, nfull + 1);        /* the KV cache lives on the device */
    else kv_alloc(m, nfull + 1);
    int *out = malloc(nfull * sizeof(int));
    memcpy(out, prompt, np * sizeof(int));
    g_temp = 0;
    double t0 = now_s();
    float *logit = g_shim_resident ? shim_step_dev(m, prompt, np, 0) : step_chunked(m, prompt, np, 0);
    double t1 = now_s();
    int len = np;
    const int force = getenv("MOTY_SHIM_FORCE") && atoi(getenv("MOTY_SHIM_FORCE"));
    double t_trace = 0;                         /* the trace rows are this file's instrument, not part of run_ref's loop */
    for (int s = 0; s < n_new; s++) {
        int best = argmax_v(logit, m->c.vocab);
        double ta = now_s();
        shim_trace_row(tf, s, logit, m->c.vocab, best);
        t_trace += now_s() - ta;
        if (!g_shim_resident) free(logit);      /* (the resident step hands out its own page-locked row) */
        out[len++] = force ? full[np + s] : best;
        if (s == n_new - 1) break;
        logit = shim_step_any(m, &out[len-1], 1, len-1);
    }
    double t2 = now_s();
    fclose(tf);
    printf("C engine : "); for (int i = np; i < nfull; i++) printf("%d ", out[i]);
    const double td = t2 - t1 - t_trace;        /* step + argmax per token, as in runtime/rt_gen_loop.h:46-84 */
    printf("\nprefill %d tok %.4f s %.2f tok/s | decode %d tok %.4f s %.2f tok/s (writing the trace rows took another %.4f s)\n",
           np, t1 - t0, np / (t1 - t0), n_new - 1, td, (n_new - 1) / td, t_trace);
    json_free(ref); free(buf); free(prompt); free(full); free(out);
    return 0;
}

int main(int argc, char **argv) {
    (void)argc;
    omp_hot_tune(argv);
    const char *th_ = getenv("THREADS");
    if (th_ && atoi(th_) > 0) moty_par_set_threads(atoi(th_));
    RunEnv e;
    if (!parse_env(&e)) return 1;
    Model m;
    if (getenv("MMAP")) g_st_map = atoi(getenv("MMAP"));
    model_init_ex(&m, e.snap, e.qbits, e.budget, e.maxctx);
    banner(&m);
    ENGINE_POST_INIT(&m);
    const char *cu = getenv("MOTY_CUDA");
    if (cu && atoi(cu) > 0) {
        int dev = getenv("MOTY_GPU") ? atoi(getenv("MOTY_GPU")) : 0;
        double t0 = now_s();
        moty_hw_cuda_open(&dev, 1);
        int n = shim_attach_model(&m, dev);
        long long bytes; moty_hw_cuda_stats(NULL, &bytes, NULL);
        fprintf(stderr, "[cuda] %d matrices on GPU %d, %.1f MB, attached in %.2f s\n", n, dev, bytes / 1048576.0, now_s() - t0);
        if (atoi(cu) >= 2) { g_shim_resident = 1; g_sd.dev = dev; }
    }
    const char *refpath = getenv("REF");
    if (!refpath) { fprintf(stderr, "set REF=<ref.json> ({\"prompt_ids\":[..],\"full_ids\":[..]})\n"); return 1; }
    const char *trace = getenv("MOTY_SHIM_TRACE");
    if (g_shim_resident && !(trace && *trace)) { fprintf(stderr, "MOTY_CUDA=2 runs through MOTY_SHIM_TRACE=<file>\n"); return 1; }
    int rc = trace && *trace ? shim_run_trace(&m, refpath, trace) : run_ref(&m, refpath);
    if (cu && atoi(cu) > 0) {
        long long calls; moty_hw_cuda_stats(NULL, NULL, &calls);
        fprintf(stderr, "[cuda] %lld mat_apply calls served by the GPU\n", calls);
    }
    return rc;
}
