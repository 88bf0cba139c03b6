/* ref_shim_gemma.c -- the reference's gemma engine as one translation unit (the way tests/gemma_tests.c includes
 * it), compiled into oracle/_ref beside ref_shim.c so that the test-suite can call functions that are static in
 * engines/gemma.c.  TEST INFRASTRUCTURE ONLY; no arithmetic of its own: every number comes out of a reference function.
 *   gelu_tanh        engines/gemma.c:389-391   (GeGLU activation of mlp(), :392-401)
 *   gnorm_row        engines/gemma.c:279-284   (RMS norm with (1 + w) or w gains)
 *   gemma_rope_head  engines/gemma.c:287-297   (p-RoPE on pairs (j, j + hd/2))
 */
#define GEMMA_TEST                      /* engines/gemma.c:544: no main() from the engine */
#include "engines/gemma.c"

/* g[i] = gelu_tanh(g[i]) * u[i], the element step of gemma's mlp() (engines/gemma.c:398) */
void refshim_gemma_gelu_mul(float *g, const float *u, int64_t n) {
    for (int64_t i = 0; i < n; i++) g[i] = gelu_tanh(g[i]) * u[i];
}

void refshim_gemma_gnorm_row(int zc_norm, float eps, float *out, const float *x, const float *w, int D) {
    Cfg c; memset(&c, 0, sizeof c);
    c.zc_norm = zc_norm; c.eps = eps;
    gnorm_row(&c, out, x, w, D);
}

void refshim_gemma_rope_head(float *x, int pos, float theta, int hd, int rot_angles) {
    gemma_rope_head(x, pos, theta, hd, rot_angles);
}
