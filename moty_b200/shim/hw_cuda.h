/* hw_cuda.h -- the CUDA backend seam of moty's hw layer.  The reference reserves hw/hw_cuda.h behind its
 * compile-time opt-in HW_CUDA (hw/hw.h:153-154, hw/hw_impl.h:62-63), but that placeholder only holds a plan and an
 * #error; this shim does not go through the hw tier selection at all: it rides the per-matrix hook of
 * moty_mat_apply, so it builds without HW_CUDA and leaves every CPU kernel in place for the formats it does not carry.
 *
 * Everything here is host C and belongs to the reference's side of the boundary: it converts between
 * the reference's types (Mat, moty_fail_code) and the C ABI of libmoty_cuda.so (include/moty_cuda.h).
 * A maintainer drops hw_cuda.c/.h into c/hw and links -lmoty_cuda.
 */
#ifndef MOTY_HW_CUDA_H
#define MOTY_HW_CUDA_H
#include "nn/nn_mat.h"

/* moty_cuda_init on the given devices (NULL/0 = device 0) and install the mat_apply hook
 * (moty_nn_set_stream_fn, nn/nn_mat.h:28-29, nn/mat.c:12-13,71).  A failure is fatal
 * (moty_fail_code): there is no CPU fallback once the backend was asked for. */
void moty_hw_cuda_open(const int *devs, int n);
/* Upload one loaded matrix and store its device handle in w->sh; from then on moty_mat_apply(…, w, S)
 * runs on the GPU.  Call right after load_mat_bits / load_mat_r4 (runtime/rt_model_load.h:85-177) and
 * after the tied-head aliasing (:440-464).  Formats the backend does not carry (f32, int2, K-quants)
 * are left alone and stay on the CPU path.  Returns 1 when the matrix went to the GPU. */
int moty_hw_cuda_attach(Mat *w, int device);
/* free the device copy (eng_close, runtime/runtime.h:335-340) */
void moty_hw_cuda_detach(Mat *w);
void moty_hw_cuda_close(void);
/* counters for a summary line: matrices attached, bytes resident, hook calls served */
void moty_hw_cuda_stats(int *n_mats, long long *bytes, long long *calls);
#endif
