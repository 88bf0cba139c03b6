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
 *   MOTY_GPU=<ordinal>                                            another GPU
 *   MOTY_SHIM_TRACE=<file>  instead of run_ref's summary: the same greedy loop (runtime/rt_gen_loop.h:46-84)
 *       with prefill and decode timed apart and one line per generated token written to <file>:
 *       "<step> <token id> <top-1 logit bits> <top-2 logit bits> <FNV-1a hash of the whole logit row>",
 *       so that two runs can be compared logit row by logit row without storing 152 k floats per step.
 */
#define QWEN_TEST                     /* engines/qwen.c:780: no main() from the engine */
#include "engines/qwen.c"
#include "hw_cuda.h"

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

static uint64_t shim_fnv(const void *p, size_t n) {
    const unsigned char *b = p; uint64_t h = 1469598103934665603ULL;
    for (size_t i = 0; i < n; i++) { h ^= b[i]; h *= 1099511628211ULL; }
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
    kv_alloc(m, nfull + 1);
    int *out = malloc(nfull * sizeof(int));
    memcpy(out, prompt, np * sizeof(int));
    g_temp = 0;
    double t0 = now_s();
    float *logit = step_chunked(m, prompt, np, 0);
    double t1 = now_s();
    int len = np;
    for (int s = 0; s < n_new; s++) {
        int best = argmax_v(logit, m->c.vocab);
        shim_trace_row(tf, s, logit, m->c.vocab, best);
        free(logit);
        out[len++] = best;
        if (s == n_new - 1) break;
        logit = step(m, &out[len-1], 1, len-1);
    }
    double t2 = now_s();
    fclose(tf);
    printf("C engine : "); for (int i = np; i < nfull; i++) printf("%d ", out[i]);
    printf("\nprefill %d tok %.4f s %.2f tok/s | decode %d tok %.4f s %.2f tok/s\n",
           np, t1 - t0, np / (t1 - t0), n_new - 1, t2 - t1, (n_new - 1) / (t2 - t1));
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
    }
    const char *refpath = getenv("REF");
    if (!refpath) { fprintf(stderr, "set REF=<ref.json> ({\"prompt_ids\":[..],\"full_ids\":[..]})\n"); return 1; }
    const char *trace = getenv("MOTY_SHIM_TRACE");
    int rc = trace && *trace ? shim_run_trace(&m, refpath, trace) : run_ref(&m, refpath);
    if (cu && atoi(cu) > 0) {
        long long calls; moty_hw_cuda_stats(NULL, NULL, &calls);
        fprintf(stderr, "[cuda] %lld mat_apply calls served by the GPU\n", calls);
    }
    return rc;
}
