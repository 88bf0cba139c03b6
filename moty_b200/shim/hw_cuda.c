/* hw_cuda.c -- reference-side shim between moty's Mat / mat_apply and libmoty_cuda.so.
 *
 * The reference already has both seams this needs and neither is touched:
 *   - Mat carries an opaque pointer `sh` that moty_mat_apply tests before its format switch, diverting
 *     the call to a hook installed with moty_nn_set_stream_fn (nn/nn_mat.h:18-30, nn/mat.c:12-13,70-71);
 *   - failures go through moty_fail_code (nn/fail.h:37): fatal in the CLI engines, a moty_status in
 *     library mode.
 * The device handle lives in `sh`; the hook is one call into the C ABI with host pointers.
 */
#include "hw_cuda.h"
#include "nn/fail.h"
#include "nn/nn_matmul.h"      /* NN_QROW_MAX */
#include "moty_cuda.h"
#include <stdlib.h>
#include <string.h>

/* The library reproduces the integer paths: IDOT=1 for int8 rows (the default, nn/matmul.c:52-53) and
 * IDOT4=1 for the two int4 row formats (opt-in, nn/matmul.c:77,171).  With the other setting of a knob
 * the reference computes an f32 product instead; those matrices stay on the CPU -- except the grouped int4
 * layout, whose f32 x int4 product the library has too (to f32 rounding, not bit for bit). */
static int env_is(const char *k, int dflt) { const char *e = getenv(k); return e && *e ? atoi(e) : dflt; }

static int g_mats;
static long long g_bytes, g_calls;

/* The engine's activations live in malloc'd buffers that come and go (falloc / free around every block), which the
 * library can only serve with copy-engine transfers from pageable memory.  Decode-sized calls (a few rows) go through
 * one pair of page-locked staging buffers instead: with pinned buffers at both ends the library moves the bytes by
 * kernels, waits on a flag word, and replays a repeated (matrix, buffers) call as one CUDA graph -- the two memcpys
 * here cost less than what that saves (MOTY_SHIM_STAGE=0: hand the engine's own pointers through). */
static float *g_xs, *g_ys;
static size_t g_xs_cap, g_ys_cap;
static int g_stage = -1;

static int stage_grow(float **p, size_t *cap, size_t bytes) {
    if (bytes <= *cap) return 0;
    if (*p) moty_cuda_host_free(*p);
    *p = NULL; *cap = 0;
    void *q = NULL;
    if (moty_cuda_host_alloc(&q, bytes + bytes / 2 + 4096) != 0) return -1;
    *p = q; *cap = bytes + bytes / 2 + 4096;
    return 0;
}

static void cuda_apply(float *y, const float *x, const struct Mat *w, int S) {
    g_calls++;
    if (g_stage < 0) g_stage = env_is("MOTY_SHIM_STAGE", 1);
    const size_t xb = (size_t)S * w->I * 4, yb = (size_t)S * w->O * 4;
    if (g_stage && S <= 8 && stage_grow(&g_xs, &g_xs_cap, xb) == 0 && stage_grow(&g_ys, &g_ys_cap, yb) == 0) {
        memcpy(g_xs, x, xb);
        if (moty_cuda_mat_apply((MotyCudaMat *)w->sh, g_ys, g_xs, S) != 0)
            moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] mat_apply %dx%d S=%d: %s\n", w->O, w->I, S, moty_cuda_last_error());
        memcpy(y, g_ys, yb);
        return;
    }
    if (moty_cuda_mat_apply((MotyCudaMat *)w->sh, y, x, S) != 0)
        moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] mat_apply %dx%d S=%d: %s\n", w->O, w->I, S, moty_cuda_last_error());
}

void moty_hw_cuda_open(const int *devs, int n) {
    if (moty_cuda_init(devs, n) != 0)
        moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] init: %s\n", moty_cuda_last_error());
    /* grouped int4: the integer product with IDOT4=1, the f32 x int4 product without (the reference's default); the
     * library takes the f32 product by itself for the row lengths the integer one does not cover (nn/matmul.c:172) */
    moty_cuda_set_i4g_float_path(env_is("IDOT4", 0) ? 0 : 1);
    moty_nn_set_stream_fn(cuda_apply);
}

int moty_hw_cuda_attach(Mat *w, int device) {
    MotyCudaMat *h = NULL;
    int rc;
    if (w->sh || w->O <= 0 || w->I <= 0) return 0;
    switch (w->fmt) {
    case WF_I8:
        if (!w->q || !w->qs || w->I > NN_QROW_MAX || !env_is("IDOT", 1)) return 0;   /* longer rows take the f32 path (nn/matmul.c:54) */
        rc = moty_cuda_upload_mat(&h, MOTY_WF_I8, w->q, w->qs, w->O, w->I, device); break;
    case WF_Q4R4:
        if (!w->q4 || !w->s16) return 0;
        rc = moty_cuda_upload_mat(&h, MOTY_WF_Q4R4, w->q4, w->s16, w->O, w->I, device); break;
    case WF_Q8R4:                                                       /* its int8 codes live in q4 too */
        if (!w->q4 || !w->s16) return 0;
        rc = moty_cuda_upload_mat(&h, MOTY_WF_Q8R4, w->q4, w->s16, w->O, w->I, device); break;
    case WF_I4:
        if (!w->q4 || !w->qs || w->I > NN_QROW_MAX || !env_is("IDOT4", 0)) return 0;
        rc = moty_cuda_upload_mat(&h, MOTY_WF_I4, w->q4, w->qs, w->O, w->I, device); break;
    case WF_I4G:                                                        /* either product of nn/matmul.c:164-253: see moty_hw_cuda_open */
        if (!w->q4 || !w->qs || w->gs != 32 || w->I % 32) return 0;
        rc = moty_cuda_upload_mat(&h, MOTY_WF_I4G, w->q4, w->qs, w->O, w->I, device); break;
    default:
        return 0;                                                       /* stays on the CPU path */
    }
    if (rc != 0)
        moty_fail_code(MOTY_FAIL_GENERIC, "[cuda] upload %dx%d fmt %d: %s\n", w->O, w->I, w->fmt, moty_cuda_last_error());
    w->sh = h;
    g_mats++; g_bytes += moty_cuda_mat_bytes(h);
    return 1;
}

void moty_hw_cuda_detach(Mat *w) {
    if (!w->sh) return;
    moty_cuda_free_mat((MotyCudaMat *)w->sh);
    w->sh = NULL;
}

void moty_hw_cuda_close(void) {
    moty_nn_set_stream_fn(NULL);
    if (g_xs) moty_cuda_host_free(g_xs);
    if (g_ys) moty_cuda_host_free(g_ys);
    g_xs = g_ys = NULL; g_xs_cap = g_ys_cap = 0;
    moty_cuda_shutdown();
}

void moty_hw_cuda_stats(int *n_mats, long long *bytes, long long *calls) {
    if (n_mats) *n_mats = g_mats;
    if (bytes) *bytes = g_bytes;
    if (calls) *calls = g_calls;
}
