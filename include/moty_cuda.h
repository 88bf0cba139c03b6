/* moty_cuda.h -- C ABI of the B200 (sm_100a) backend for moty's quantized-matmul path.
 *
 * One shared library, libmoty_cuda.so.  Plain C types only: pointers, ints,
 * opaque handles.  Every function returns 0 on success and a negative
 * MOTY_CUDA_E* code on failure (moty_cuda_last_error() holds the message); the
 * library never falls back to the CPU and never longjmps.  Calls are serial per
 * process, like the reference drivers they replace (those keep function-level
 * static scratch: nn/matmul.c:55-58, 370).
 *
 * Naming follows the call sites of moty's absent CUDA backend
 * (engines/glm.c:244, 797-809, 5709: moty_cuda_init / _tensor_upload / _matmul).
 * "Replaces" below names the reference function (moty source tree, directory
 * c/) whose results each entry reproduces.
 *
 * Pointer suffix convention: plain entries take HOST pointers for activations
 * and results (they copy in and out on the library's stream and return after
 * the result is in host memory); *_dev entries take DEVICE pointers, enqueue on
 * `stream` (a cudaStream_t passed as void*, NULL = the library's own stream; a caller whose work is on CUDA's
 * default stream passes cudaStreamLegacy or cudaStreamPerThread, not 0) and
 * return without synchronising.  *_dev entries that take no matrix or layer handle run on the GPU that owns
 * their first device pointer (which must have been initialised).  Every entry leaves the caller's current CUDA
 * device as it found it.
 *
 * CUDA graphs: the *_dev entries can be captured, with two rules.  The per-device scratch grows on demand (which
 * frees and reallocates): run the largest call of the pipeline once, then moty_cuda_scratch_freeze(device, 1), then
 * capture.  And the first call of any entry on a device may set kernel attributes: make it before the capture.
 */
#ifndef MOTY_CUDA_H
#define MOTY_CUDA_H
#include <stdint.h>
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

/* weight formats: the values of the WF_* enum in hw/hw.h:53 */
enum { MOTY_WF_F32 = 0, MOTY_WF_I8 = 1, MOTY_WF_I4 = 2, MOTY_WF_I4G = 4, MOTY_WF_Q4R4 = 7, MOTY_WF_Q8R4 = 8 };
/* activations between the two halves of an FFN (hw/hw_ops.h:19-21, engines/gemma.c:389-391) */
enum { MOTY_ACT_SILU = 0, MOTY_ACT_GELU_TANH = 1 };

enum {
    MOTY_CUDA_OK = 0,
    MOTY_CUDA_EINIT = -1,      /* library not initialised / device not in the set */
    MOTY_CUDA_EARG = -2,       /* bad argument (shape, format, NULL) */
    MOTY_CUDA_ECUDA = -3,      /* a CUDA call failed */
    MOTY_CUDA_ENOMEM = -4,     /* device allocation failed */
    MOTY_CUDA_ELIMIT = -5,     /* size beyond what the entry point supports */
    MOTY_CUDA_EKERNEL = -6     /* a kernel reported an internal error (bounded wait expired) */
};

typedef struct MotyCudaMat MotyCudaMat;   /* one weight matrix resident on one GPU */
typedef struct MotyCudaMoe MotyCudaMoe;   /* one MoE layer: router + resident experts */

/* ---- lifecycle -------------------------------------------------------- */

/* Select the GPUs (ndev >= 1 device ordinals; NULL/0 = device 0), create one
 * stream and the scratch arenas per device.  Precedent: moty_cuda_init(devices,
 * ndev) at engines/glm.c:5701-5709. */
int moty_cuda_init(const int *devices, int ndev);
void moty_cuda_shutdown(void);
const char *moty_cuda_last_error(void);
/* SM count of an initialised device, <0 on error */
int moty_cuda_sm_count(int device);
/* block until everything enqueued on the library's stream of `device` is done */
int moty_cuda_sync(int device);

/* Status of the kernels with bounded waits.  Nothing in this library waits without a limit (mbarrier waits of the
 * tensor-core GEMM and of the bulk-copy fed Q4R4/Q8R4 decode kernels, the grid barrier of the one-launch MoE/FFN
 * decode kernels); a wait that runs out makes its kernel set a device error word and return with an incomplete
 * result.  The host-pointer entries check the words themselves and return MOTY_CUDA_EKERNEL.  A device-resident
 * pipeline (the *_dev entries return before anything ran) calls this instead, e.g. once per generated token: it
 * waits for `stream` (NULL = the library's), returns 0 when no wait expired since the last check, else clears the
 * words, puts the grid-barrier counters back to zero and returns MOTY_CUDA_EKERNEL (last_error names the kernel
 * class).  It also reports a device-side position of moty_cuda_attn_core_posdev that left [0, pos_max] (the kernels
 * clamp it instead of writing past the KV cache).  The reference's kernels cannot fail (hw/hw.h:58-124 return no status); this is the GPU-side addition. */
int moty_cuda_kernel_status(int device, void *stream);
/* Diagnostic: enqueue a tiny kernel that runs the give-up path of one wait class on purpose -- the production wait
 * function on something nobody completes, with a limit well under a millisecond; it polls, gives up, sets the
 * error word and exits (no fault, no trap, no hang).  which: 0 = GEMM pipeline wait, 1 = grid barrier (leaves the
 * barrier counters inconsistent, as a real expiry would), 2 = bulk-copy wait.  moty_cuda_kernel_status must then
 * report MOTY_CUDA_EKERNEL once and the next ordinary call must succeed. */
int moty_cuda_selftest_expire_wait(int device, int which, void *stream);
/* The per-device scratch of the drivers grows on demand, which frees and reallocates it.  A captured CUDA graph
 * holds the addresses it was captured with, so: run the largest call once, then freeze (on = 1) before capturing;
 * from then on a call that would need more scratch returns MOTY_CUDA_ELIMIT instead of moving the buffers under
 * the graph.  on = 0 lifts the freeze (graphs captured before must then be dropped).  No reference counterpart:
 * its drivers grow function-level static scratch with malloc (nn/matmul.c:55-58). */
int moty_cuda_scratch_freeze(int device, int on);
/* CUDA graphs for a caller that does not link the CUDA runtime itself (the reference is plain C): everything the *_dev
 * entries enqueue on `stream` (NULL = the library's) between graph_begin and graph_end is captured instead of run;
 * graph_launch replays it on that stream.  Rules: run the sequence once before capturing it (scratch, kernel
 * attributes); between begin and end call only *_dev entries that enqueue work (no uploads from pageable memory, no
 * downloads, no kernel_status); take positions from the device (moty_cuda_attn_core_posdev) and feed token ids and
 * positions with moty_cuda_dev_upload before each launch.  graph_end freezes the scratch (as scratch_freeze does) until
 * the graph is freed.  No reference counterpart. */
typedef struct MotyCudaGraph MotyCudaGraph;
int moty_cuda_graph_begin(int device, void *stream);
int moty_cuda_graph_end(MotyCudaGraph **out, int device, void *stream);
int moty_cuda_graph_launch(MotyCudaGraph *g);
int moty_cuda_graph_free(MotyCudaGraph *g);

/* Device memory for a C host that keeps its activations on the GPU between *_dev entries without the CUDA headers
 * (the reference is plain C): allocate, free, copy in (enqueued on `stream`, NULL = the library's; returns at once)
 * and copy out (returns when the bytes are in host memory).  Thin wrappers of cudaMalloc / cudaFree / cudaMemcpyAsync. */
int moty_cuda_dev_alloc(void **p, size_t bytes, int device);
int moty_cuda_dev_free(void *p);
int moty_cuda_dev_upload(void *dst_dev, const void *src, size_t bytes, int device, void *stream);
int moty_cuda_dev_download(void *dst, const void *src_dev, size_t bytes, int device, void *stream);

/* pinned host memory for callers that want asynchronous copies on the plain
 * (host-pointer) entries; ordinary malloc'd memory works too, only slower */
int moty_cuda_host_alloc(void **p, size_t bytes);
int moty_cuda_host_free(void *p);

/* ---- weights ----------------------------------------------------------
 * Replaces the host-side Mat descriptor (nn/nn_mat.h:18-25).  Layouts are the
 * reference's own, copied byte for byte:
 *   MOTY_WF_I8   codes int8 [O][I] row-major, scales f32 [O]            (nn/quant.c:12-33)
 *   MOTY_WF_Q4R4 codes uint8 [ceil(O/4)][I/32][64], scales f16 [ceil(O/4)][I/32][4]
 *                                                                         (hw/hw_q4r4.h:3-11)
 *   MOTY_WF_Q8R4 codes int8 [ceil(O/4)][I/32][128] (4 rows x 32 codes), scales as Q4R4
 *                                                                         (hw/hw_q4r4.h:92-99)
 *   MOTY_WF_I4   codes uint8 [O][(I+1)/2], scales f32 [O]               (nn/quant.c:35-55); kept on the device as
 *                the int8 codes nibble - 8 (twice the bytes): the integer path of moty_matmul_i4_s (nn/matmul.c:75-101,
 *                IDOT4=1) is the Q8_0 product over those codes, so every Q8_0 kernel serves it bit for bit;
 *                moty_cuda_mat_shape still reports MOTY_WF_I4, moty_cuda_mat_bytes the bytes held
 *   MOTY_WF_I4G  codes uint8 [O][I/2] (even element in the low nibble), scales f32 [O][I/32]: grouped int4,
 *                group size 32 (nn/quant.c:57-83); applied through the integer path of
 *                moty_matmul_i4_grouped_s (nn/matmul.c:164-197, IDOT4=1) when I % 64 == 0 and I <= 16384,
 *                else -- and always after moty_cuda_set_i4g_float_path(1) -- through its default product,
 *                f32 activations x dequantized int4 (i4g_f32_rows, nn/matmul.c:196-253)
 *   MOTY_WF_F32  codes float [O][I], scales NULL (router matrices only)
 * The hook point in the loader is right after load_mat_bits / load_mat_r4 /
 * load_embed_q8 (runtime/rt_model_load.h:85-177, 209-226). */
int moty_cuda_upload_mat(MotyCudaMat **out, int fmt, const void *codes, const void *scales,
                         int O, int I, int device);
/* rows [o0, o1) of the same host matrix: the row shard of one GPU.  For
 * MOTY_WF_Q4R4 and MOTY_WF_Q8R4 o0 must be a multiple of 4. */
int moty_cuda_upload_mat_rows(MotyCudaMat **out, int fmt, const void *codes, const void *scales,
                              int O, int I, int o0, int o1, int device);
int moty_cuda_free_mat(MotyCudaMat *m);
int64_t moty_cuda_mat_bytes(const MotyCudaMat *m);
int moty_cuda_mat_shape(const MotyCudaMat *m, int *fmt, int *O, int *I, int *device);

/* ---- the operator boundary --------------------------------------------
 * Replaces moty_mat_apply(y, x, w, S) (nn/mat.c:70-83) for the formats above:
 *   WF_I8   -> moty_matmul_q_s      (nn/matmul.c:51-66, IDOT=1 path)
 *   WF_Q4R4 -> moty_matmul_q4r4_s   (nn/matmul.c:405-433)
 *   WF_I4   -> moty_matmul_i4_s with IDOT4=1 (nn/matmul.c:75-96)
 * x is [S][I] f32, y is [S][O] f32.  Like the reference, I <= 16384 for the
 * integer paths (NN_QROW_MAX, nn/nn_matmul.h:35); larger I is MOTY_CUDA_ELIMIT.
 * Host pointers; returns with y written.  When x and y both lie in page-locked memory (moty_cuda_host_alloc,
 * cudaHostAlloc, cudaHostRegister; 16-byte aligned) and the product has no error word to report (MOTY_WF_I8 below 9
 * rows and the like), the bytes move by kernels chained to the product and the call waits on a flag word instead of
 * synchronising the stream; a call that repeats with the same matrix and buffers (a decode loop) is replayed as one
 * CUDA graph of those launches from its third occurrence on (dropped when the scratch moves or a matrix is freed).
 * Pageable buffers take copy-engine transfers.  Same results; MOTY_CUDA_HOST_KERNELS=0 in the environment forces the
 * copies. */
int moty_cuda_mat_apply(MotyCudaMat *w, float *y, const float *x, int S);
/* MOTY_WF_I4G products: 0 (default) = the integer path the reference takes with IDOT4=1 (bit-exact), 1 = the product it
 * takes without that switch, f32 x int4 with one scale multiply per group of 32 (agrees with the reference to the f32
 * rounding of a 32-term sum: its own SIMD tiers order that sum differently too).  Returns the previous value. */
int moty_cuda_set_i4g_float_path(int on);
/* MOTY_WF_Q4R4 / MOTY_WF_Q8R4 batches of five rows and more, dense and grouped (MoE prompts): 0 (default) = bit for bit
 * what moty_matmul_q4r4_s computes, which has two formulas for a group's term and picks one by the token's place in its
 * 32-token tile (hw/hw_q4r4.h:58-59 token by token, :78-81 four tokens at a time); 1 = the token-by-token formula for
 * every token: tokens the reference treats that way keep their bits, the others move by the rounding of one fused
 * multiply-add per group (about 1e-7 of the row's largest term), and the kernel sheds the second of its two
 * accumulate steps (1.2x on large batches).
 * Batches of up to four rows are not affected.  Returns the previous value. */
int moty_cuda_set_q4r4_batch_relaxed(int on);
int moty_cuda_mat_apply_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, int S, void *stream);
/* n (1..8) independent one-row products in ONE launch: y_dev[m] = mat_apply(w[m], x_dev[m], S = 1) for MOTY_WF_I8
 * matrices on one GPU with I % 16 == 0 and I <= 16384 (x_dev[m] 16-byte aligned; the pointers may repeat: the q, k, v
 * projections of a layer share their row; rows longer than 4096 values are split in K and combined exactly, as in the
 * single-matrix kernel).  Small matrices cost a launch each otherwise (1-3 MB: 0.2-0.5 us of HBM
 * time behind 4-5 us of fixed cost); here all rows of all matrices are dealt to one persistent grid.  Same bits as n
 * calls of mat_apply_dev.  w, y_dev, x_dev are HOST arrays of n pointers.  No reference counterpart (the reference
 * calls moty_mat_apply once per matrix, nn/mat.c:70). */
int moty_cuda_mat_apply_multi_dev(int n, MotyCudaMat *const *w, float *const *y_dev, const float *const *x_dev, void *stream);
/* same, also returning the int32 accumulators [S][O] of the Q8_0 path (the
 * values moty_hw_dot_i8i8 returns, hw/hw_scalar.h:8-12) for exact checks */
int moty_cuda_mat_apply_acc(MotyCudaMat *w, float *y, int32_t *acc, const float *x, int S);

/* The Q8_0 product for hosts that must not allocate (no counterpart in the
 * reference: its drivers grow static scratch with malloc).  Meant for callers
 * that own all device memory themselves, or that cannot take the device-wide
 * stall of cudaMalloc/cudaFree inside a decode loop.  All four arrays are DEVICE
 * pointers supplied by the caller: q [O][I] int8, scale [O], x [S][I], y [S][O].
 * The quantized activation rows live in a fixed array inside the library
 * (8 x 16384 bytes of codes + 8 scales per GPU, held until the process exits), so
 *   1 <= S <= 8, I a multiple of 16, 16 <= I <= 16384; anything else is
 *   MOTY_CUDA_ELIMIT.  q_dev must be 16-byte aligned (the product kernel reads weights with 128-bit loads;
 *   a sliced tensor may not be), y_dev, x_dev and scale_dev 4-byte aligned: MOTY_CUDA_EARG otherwise, before
 *   any launch.  The caller's current device is left as it was.
 * The call needs no moty_cuda_init and calls no allocating routine.  Its FIRST
 * call on a device looks up the array's device address and sets kernel
 * attributes; make that first call before any stream capture.  All calls share
 * the one array: two calls that overlap on the GPU (different streams) race;
 * calls on one stream are ordered and safe.  Results equal moty_cuda_mat_apply_dev
 * bit for bit.  `stream` NULL = the default stream. */
int moty_cuda_q8_apply_noalloc(float *y_dev, const float *x_dev, const int8_t *q_dev, const float *scale_dev,
                               int S, int I, int O, int device, void *stream);

/* HwBackend.matmul_i8 (hw/hw_backend.h:56-57) / moty_matmul_q_s with host
 * weights: uploads, runs, frees.  A correctness convenience, not a fast path. */
int moty_cuda_matmul_q_s(float *y, const float *x, const int8_t *q, const float *scale, int S, int I, int O);
/* moty_matmul_q4r4_s (nn/matmul.c:405) with host weights */
int moty_cuda_matmul_q4r4_s(float *y, const float *x, const uint8_t *q4, const uint16_t *s16, int S, int I, int O);
/* moty_matmul_i4_grouped_s (nn/matmul.c:164) with host weights, integer path (IDOT4=1), gs = 32 only */
int moty_cuda_matmul_i4_grouped_s(float *y, const float *x, const uint8_t *q4, const float *scale,
                                  int S, int I, int O, int gs);
/* moty_matmul_q8r4_s (nn/matmul.c:435-461): the int8 sibling of Q4R4 used for mixed precision
 * (tensors matched by Q8_TENSORS, runtime/rt_model_load.h:38-61); uploads per call like the two above */
int moty_cuda_matmul_q8r4_s(float *y, const float *x, const int8_t *q8, const uint16_t *s16, int S, int I, int O);

/* ---- kernels of the hw.h contract, host-callable ----------------------- */

/* moty_hw_qrow_i8 (hw/hw_quant.h:9-16) over `rows` rows of n floats:
 * q [rows][n] int8, scale [rows] f32. */
int moty_cuda_qrow_i8(const float *x, int8_t *q, float *scale, int rows, int n);
int moty_cuda_qrow_i8_dev(const float *x_dev, int8_t *q_dev, float *scale_dev, int rows, int n, void *stream);
/* moty_hw_quant_g32 (hw/hw_q4r4.h:36-45) over `rows` rows of I floats (I % 32 == 0) */
int moty_cuda_quant_g32(const float *x, int rows, int I, int8_t *xq, float *xs, int32_t *xsum);
int moty_cuda_quant_g32_dev(const float *x_dev, int rows, int I, int8_t *xq_dev, float *xs_dev,
                            int32_t *xsum_dev, void *stream);
/* moty_hw_dot_i8i8 (hw/hw_scalar.h:8-12): nrows dots of length n, w [nrows][n]
 * against one x [n]; out [nrows] int32.  A test entry: per-row host calls are
 * meaningless for speed, the GEMV/GEMM kernels use the same device code. */
int moty_cuda_dot_i8i8(const int8_t *w, const int8_t *x, int nrows, int n, int32_t *out);
/* moty_hw_dot_i4i8 (hw/hw_scalar.h:14-22), same calling shape; w4 [nrows][(n+1)/2] */
int moty_cuda_dot_i4i8(const uint8_t *w4, const int8_t *x, int nrows, int n, int32_t *out);

/* ---- router ------------------------------------------------------------
 * moty_moe_topk (runtime/moecache.c:97-111) on `rows` rows of E already
 * soft-maxed values: idx [rows][K] int32, w [rows][K] f32. */
int moty_cuda_moe_topk(const float *probs, int rows, int E, int K, int *idx, float *w, int norm_topk);
/* route_topk (nn/moe.c:27-30): softmax (hw/hw_ops.h:22-26) then top-K with
 * renormalisation.  probs_out (optional) receives the softmax [rows][E]. */
int moty_cuda_route_topk(const float *logits, int rows, int E, int K, int *idx, float *w, float *probs_out);
int moty_cuda_route_topk_dev(const float *logits_dev, int rows, int E, int K, int *idx_dev, float *w_dev,
                             float *probs_dev, int norm_topk, void *stream);

/* ---- dense FFN -----------------------------------------------------------
 * Replaces moty_nn_dense_ffn (nn/ffn.c:26-55) and the engines' mlp()
 * (engines/qwen.c:654-679 SiLU, engines/gemma.c:392-401 tanh-GeLU):
 * out = down( act(gate x) * up x ), x [S][D], out [S][D].  The intermediate
 * [S][I] never leaves the GPU. */
int moty_cuda_ffn(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act,
                  float *out, const float *x, int S);
int moty_cuda_ffn_dev(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act,
                      float *out_dev, const float *x_dev, int S, void *stream);

/* ---- MoE layer -------------------------------------------------------------
 * Replaces the MotyMoeView + ExpertCache pair (nn/moe.h:20-33, runtime/moe.h:35-54)
 * with all experts resident on the GPU, keyed by expert id (never by slot
 * pointer: the reference reuses slots on eviction, runtime/moecache.c:51-89).
 * efmt: MOTY_WF_I8 (ExpertSlot layout: g,u [I][D] int8 + f32 row scales,
 * d [D][I]) or MOTY_WF_Q4R4 (each projection in the Q4R4 block layout).
 * Experts [e_lo, e_hi) live on this GPU (expert-parallel shard); others are
 * skipped by the block entries and must be served by another rank. */
int moty_cuda_moe_create(MotyCudaMoe **out, int E, int K, int I, int D, int efmt,
                         int e_lo, int e_hi, int device);
int moty_cuda_moe_free(MotyCudaMoe *m);
/* what LoadExpertFn (runtime/moe.h:56, engines/olmoe.c:141-151) fills for one expert */
int moty_cuda_moe_upload_expert(MotyCudaMoe *m, int eid, const void *g, const void *gs,
                                const void *u, const void *us, const void *d, const void *ds);
/* The same for LFM2's int4 experts (ExpertSlot rows with ebits <= 4, nn/moe.h:12, nn/moe.c:42,99-103,138,193-198):
 * g4, u4 [I][(D+1)/2] and d4 [D][(I+1)/2] nibble rows (element 2j in the low nibble), f32 row scales.  The layer must
 * have been created with MOTY_WF_I8: the rows are expanded to the signed codes nibble - 8 on the way in, whose integer
 * dots are the reference's dot_i4i8p sums, so decode, batches and both gates give the reference's bits (the reference's
 * batch path is integer under IDOT4=1, nn/matmul.c:75-96).  Costs int8 bytes in HBM, not int4. */
int moty_cuda_moe_upload_expert_i4(MotyCudaMoe *m, int eid, const void *g4, const float *gs,
                                   const void *u4, const float *us, const void *d4, const float *ds);
/* optional router matrix [E][D]; without one the block entries need `logits` */
int moty_cuda_moe_set_router(MotyCudaMoe *m, MotyCudaMat *router);

/* LFM2's gate instead of the softmax one: route_sigmoid (nn/moe.c:10-25) -- probs = 1 / (1 + expf(-logit)), the K
 * largest probs + expert_bias (strict >, ties to the lowest index), weights = the unbiased probabilities of the picks
 * over their sum.  With on != 0 the block entries below compute moty_nn_moe_sigmoid_d1 / _batch (nn/moe.c:154,207)
 * instead of the _topk_ ones; expert_bias [E] (host) may be NULL (MotyMoeView.expert_bias, nn/moe.h:22).  int8
 * experts (ebits = 8); the reference's int4-packed expert rows (ebits <= 4, nn/moe.c:99-103) are not carried. */
int moty_cuda_moe_set_sigmoid_gate(MotyCudaMoe *m, int on, const float *expert_bias);

/* moty_nn_moe_topk_d1 (nn/moe.c:33-153): one token.  logits (optional, [E]) are
 * the router outputs; NULL = compute them with the router set above.  The K
 * weighted expert outputs are summed in selection order k = 0..K-1. */
int moty_cuda_moe_d1(MotyCudaMoe *m, float *out, const float *x, const float *logits);
/* moty_nn_moe_topk_batch (nn/moe.c:159-205): S tokens; a token's expert outputs
 * are summed in ascending expert id. */
int moty_cuda_moe_batch(MotyCudaMoe *m, float *out, const float *x, int S, const float *logits);
/* engines/olmoe.c:219-244: S tokens, each summed in selection order, with the
 * config's norm_topk flag. */
int moty_cuda_olmoe_moe(MotyCudaMoe *m, float *out, const float *x, int S, const float *logits, int norm_topk);
/* device-pointer form of the three above.  order: 0 = selection order (d1 /
 * olmoe), 1 = ascending expert id (batch).  idx_dev/w_dev (optional) return the
 * routing [S][K].  partial != 0: only this GPU's experts contribute and the
 * result is a partial sum to be combined across ranks. */
int moty_cuda_moe_apply_dev(MotyCudaMoe *m, float *out_dev, const float *x_dev, int S,
                            const float *logits_dev, int order, int norm_topk,
                            int *idx_dev, float *w_dev, void *stream);

/* One token through a routed layer normally takes a decode path that streams the
 * selected experts once.  int8 experts with the softmax gate: two launches chained by
 * programmatic dependent launch (route + gate/up + SiLU, then down + ordered sum);
 * the expert-parallel decode entries below use ONE cooperative launch instead (router,
 * gate/up, a bounded grid barrier, down), which also holds their exchange.  Q4R4
 * experts: one cooperative launch.  Same arithmetic, same bits as the general grouped
 * path that batches use.  This switch lets a test run them all and compare:
 * 1 = best decode path (default), 2 = the split decode path (separate router /
 * gate-up / down launches, both formats), 0 = the grouped path, 3 = as 1 with the
 * cooperative kernel wherever one exists: int8 decode tokens, and a one-token dense
 * int8 SiLU FFN block (moty_cuda_ffn[_dev]) run as a one-expert layer instead of its
 * default two chained launches (gate + up + activation, then down).  Returns the
 * previous value; no reference counterpart.  If a cooperative kernel's barrier wait
 * ever expires (a fraction of a second), the host-pointer entries return
 * MOTY_CUDA_EKERNEL. */
int moty_cuda_set_moe_fast_path(int on);
/* Batches through int8 experts (moty_nn_moe_topk_batch, nn/moe.c:159-205) run their grouped products on the tensor
 * cores (tcgen05, gate+up+SiLU in one pass) when the experts see 8 or more routed rows each on average, else on
 * mma.sync tiles that stream the weights once.  Same arithmetic, same bits.  This switch lets a test compare the two:
 * 1 = as described (default), 0 = mma.sync tiles always.  Returns the previous value; no reference counterpart. */
int moty_cuda_set_moe_batch_path(int tensor_core);

/* Expert-parallel building blocks (no reference counterpart: the reference is one
 * process).  Arithmetic is that of the block entries above, cut at the exchange.
 * moe_experts_dev: P activation rows x_rows [P][D], each with ONE expert id
 * eid [P] (the rows a peer routed here); h [P][D] receives that expert's output
 * down(silu(gate x) * up x) per row, zeros for experts not resident on this GPU.
 * Per-row results equal what nn/moe.c:195-199 computes for that row. */
int moty_cuda_moe_experts_dev(MotyCudaMoe *m, float *h_dev, const float *x_rows_dev, const int *eid_dev,
                              int P, void *stream);
/* One token, expert-parallel decode: like moe_apply_dev with S = 1 and selection order, and additionally
 * rows_dev [K][D] receives every selected expert's OWN output row h_k (before the routing weight): the row itself
 * for experts resident on this GPU, zeros for the others.  Every rank routes the same token redundantly (same
 * logits -> same top-K), so the ranks' row tables have disjoint non-zero rows; their element-wise sum (an
 * all-reduce, x + 0 is exact) is the full table on every rank, and moe_combine_dev(order 0) then adds the K rows
 * in selection order exactly as nn/moe.c:146-149 does -- the result has the one-GPU bits.  out_dev [D] receives
 * this GPU's partial sum.  Needs a layer shape the one-launch decode kernels take (MOTY_CUDA_ELIMIT otherwise). */
int moty_cuda_moe_d1_rows_dev(MotyCudaMoe *m, float *rows_dev, float *out_dev, const float *x_dev,
                              const float *logits_dev, int norm_topk, int *idx_dev, float *w_dev, void *stream);
/* The same expert-parallel decode with the exchange done by the library's own kernels over peer memory (NVLink)
 * instead of a collective: tables[r] / flags[r] (host arrays of `world` DEVICE pointers, r = rank) are every rank's
 * row tables (2 * K * D floats each: two tables used alternately) and flag words (`world` u32 each, zero before the
 * first call) in memory that every GPU of the group can address (peer access or symmetric memory).  The decode
 * kernel stores the rows of this GPU's experts straight into all ranks' tables; a second launch signals each peer
 * (fence + one release store into the peer's word for this rank), waits -- BOUNDED, about a second; on expiry the
 * error word is set, nothing is written and moty_cuda_kernel_status reports it -- until all ranks' rows of step
 * `epoch` have arrived, and adds the K rows in selection order: the one-GPU bits.  epoch: 1, 2, 3, ... the same on
 * every rank, one per call.  1 <= world <= 8; one rank per GPU (ranks that wait for each other must never share one). */
int moty_cuda_moe_d1_peer_dev(MotyCudaMoe *m, float *out_dev, const float *x_dev, const float *logits_dev, int norm_topk,
                              void *const *tables, void *const *flags, int world, int rank, unsigned epoch, void *stream);
/* moe_combine_dev: out[s] = sum over the token's K selections of w[s][k] * h[s*K+k],
 * one fused multiply-add per step from 0, in selection order (order 0,
 * nn/moe.c:146-149) or ascending expert id (order 1, nn/moe.c:200-202). */
int moty_cuda_moe_combine_dev(float *out_dev, const float *h_dev, const float *w_dev, const int *idx_dev,
                              int S, int K, int D, int order, void *stream);

/* ---- greedy token ----------------------------------------------------------
 * moty_argmax_v (nn/sample.c:9-13): first index of the maximum of v [n]. */
int moty_cuda_argmax(const float *v, int n, int *out);
int moty_cuda_argmax_dev(const float *v_dev, int n, int *out_dev, void *stream);
/* The lm_head and the greedy pick in one call (moty_nn_head_apply without the speculative head,
 * nn/head.c:134-135, followed by moty_argmax_v, nn/sample.c:9-13, as the engines' decode step does):
 * ids [S] receives the first index of each row's maximum; the S x O logits stay on the device unless
 * `logits` (host, [S][O]) / `logits_dev` is given.  x: [S][I].  Results equal mat_apply + argmax. */
int moty_cuda_head_argmax(MotyCudaMat *head, const float *x, int S, int *ids, float *logits);
int moty_cuda_head_argmax_dev(MotyCudaMat *head, const float *x_dev, int S, int *ids_dev, float *logits_dev, void *stream);

/* ---- the f32 steps of a decoder layer around the matmuls (device pointers) ----
 * So that a layer's activations can stay on the device between the entries above.
 * rmsnorm: moty_rmsnorm_row per row (nn/norm.c:7, hw/hw_ops.h:14-18): mean of squares in double,
 *          out = x * (1 / sqrtf((float)(ms / D) + eps)) * w;  x, out [S][D], w [D] (all device).
 * add:     moty_hw_add (hw/hw_ops.h:30-32): y[i] += x[i].
 * embed_rows: embed_row for an int8 table (runtime/rt_model_load.h:656-660; the tied lm_head uploaded as
 *          MOTY_WF_I8 [vocab][D]): out[s][i] = (qs[id] * scale) * (float)q[id][i], ids_dev int32 [S] on the device. */
int moty_cuda_rmsnorm_dev(float *out_dev, const float *x_dev, const float *w_dev, int S, int D, float eps, void *stream);
int moty_cuda_add_dev(float *y_dev, const float *x_dev, long long n, void *stream);
/* add_rmsnorm: the residual add followed by the next norm, one launch: x += t, then out = rmsnorm(x) with gains w
 * (same results as add_dev followed by rmsnorm_dev). */
int moty_cuda_add_rmsnorm_dev(float *x_dev, const float *t_dev, float *out_dev, const float *w_dev, int S, int D,
                              float eps, void *stream);
/* normadd_rmsnorm: the sandwich step of engines/gemma.c:468-474 / :478-482, one launch: x += rmsnorm(t) with gains
 * g_t (the post-block norm, done in place on the block's output there), then -- when out_dev is not NULL --
 * out = rmsnorm(x) with gains g_x (the norm that opens the next block).  The gains are the multipliers themselves:
 * pass 1 + w for a zero-centred checkpoint (gnorm_row, engines/gemma.c:279-284).  t is left as it was. */
int moty_cuda_normadd_rmsnorm_dev(float *x_dev, const float *t_dev, const float *g_t_dev, float *out_dev, const float *g_x_dev,
                                  int S, int D, float eps, void *stream);
/* The same residual step and norm folded into the one-token product or FFN block that consumes them (one launch less
 * per fold; every CTA of the consumer forms the row for itself):
 *   xout = x + t                      when g_t_dev is NULL   (add_rmsnorm_dev),
 *   xout = x + rmsnorm(t) * g_t       otherwise              (normadd_rmsnorm_dev, gemma's sandwich),
 *   row  = rmsnorm(xout) * g_x,   then   y = W * row   (mat_apply_resnorm_dev)   or   out = FFN(row)   (ffn_resnorm_dev).
 * xout_dev must overlap neither x_dev nor t_dev (one CTA writes xout while every other still reads x and t;
 * MOTY_CUDA_EARG otherwise); x_dev and t_dev 16-byte aligned.  MOTY_WF_I8 matrices whose rows (I of W; D of gate/up)
 * are a multiple of 16 and at most 4096 values: mat_addnorm_supported / ffn_resnorm_supported say whether they qualify.
 * Same bits as the separate entries one after the other.  mat_apply_addnorm_dev is mat_apply_resnorm_dev without g_t. */
int moty_cuda_mat_addnorm_supported(const MotyCudaMat *w);
int moty_cuda_mat_apply_addnorm_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, const float *t_dev,
                                    float *xout_dev, const float *gain_dev, float eps, void *stream);
int moty_cuda_mat_apply_resnorm_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, const float *t_dev,
                                    const float *g_t_dev, float *xout_dev, const float *g_x_dev, float eps, void *stream);
int moty_cuda_ffn_resnorm_supported(const MotyCudaMat *gate, const MotyCudaMat *up);
int moty_cuda_ffn_resnorm_dev(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act, float *out_dev,
                              const float *x_dev, const float *t_dev, const float *g_t_dev, float *xout_dev,
                              const float *g_x_dev, float eps, void *stream);
int moty_cuda_embed_rows_dev(MotyCudaMat *embed, float *out_dev, const int *ids_dev, int S, float scale, void *stream);

/* ---- attention core between the projections --------------------------------
 * attn_tail of nn/attn.c:29-74 without the q/k/v/o projections (those are mat_apply calls) and
 * without the optional output gate: QK-norm (moty_rmsnorm_row per head with qn / kn [head_dim],
 * NULL = none) and RoPE (moty_rope_head: half-split over the first `rot` dimensions, base theta),
 * K and V rows stored at positions pos_base .. pos_base+S-1 of the layer's cache (f32, or with
 * kv8 != 0 int8 rows with one qrow_i8 scale per head and position, moty_kv_store_row), then per
 * head and token the scores against positions 0..pos, softmax and accumulation
 * (moty_att_scores_* / moty_softmax_row / moty_att_accum_*).  One MotyCudaAttn per layer holds the
 * KV cache of max_t positions on the device (MotyCommon's K/V or K8/V8/Ks/Vs of that layer).
 * q [S][H*hd], k, v [S][KV*hd] -> ctx [S][H*hd].  f32 arithmetic with libm calls whose summation
 * order already differs between the reference's CPU tiers: results agree to a few 1e-6, not bit
 * for bit.  The _dev entry norms and rotates q_dev and k_dev in place, as the reference does. */
typedef struct MotyCudaAttn MotyCudaAttn;
int moty_cuda_attn_create(MotyCudaAttn **out, int n_heads, int n_kv_heads, int head_dim, int rot, float theta,
                          float eps, const float *qn, const float *kn, int max_t, int kv8, int device);
/* gemma's attention (engines/gemma.c:299-386 without the projections, shared-KV layers and k_eq_v): qn / kn / vn are
 * the norm MULTIPLIERS per head dimension (1 + w with the engine's default zc_norm, w with GEMMA_NORM_PLAIN, :279-284;
 * vn = the value norm, NULL = none), p-RoPE on pairs (j, j + head_dim/2) for j < rot_pairs with frequency
 * theta^(-2j/head_dim) (:287-297; sliding layers rotate all head_dim/2 pairs), scores scaled by `scale`
 * (1/sqrt(query_pre_attn_scalar), :363; 0 = 1/sqrt(head_dim)), and with window > 0 a token attends to positions
 * max(0, pos - window + 1) .. pos only (:373; 0 = a global layer).  The handle is then used with the core entries below. */
int moty_cuda_attn_create_gemma(MotyCudaAttn **out, int n_heads, int n_kv_heads, int head_dim, int rot_pairs, float theta,
                                float eps, const float *qn, const float *kn, const float *vn, int window, float scale,
                                int max_t, int kv8, int device);
int moty_cuda_attn_free(MotyCudaAttn *a);
int moty_cuda_attn_core(MotyCudaAttn *a, float *ctx, const float *q, const float *k, const float *v, int S, int pos_base);
int moty_cuda_attn_core_dev(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev,
                            int S, int pos_base, void *stream);
/* The same with the first position read from a device int at run time: a decode step captured once into a CUDA graph
 * is replayed while the position moves.  pos_max = the largest value *pos_dev may take (it sizes the launch);
 * pos_max + S must fit the cache.  Results equal attn_core_dev at the same position.  With S = 1 the norm, the rotation
 * and the cache store happen inside the scores launch (one launch less per decode step) and q_dev, k_dev are left as
 * they came instead of being rotated in place. */
int moty_cuda_attn_core_posdev(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev,
                               int S, const int *pos_dev, int pos_max, void *stream);
/* the last step of the gated variant (moty_nn_attention_gated, nn/attn.c:68-69): ctx[i] *= 1 / (1 + expf(-gate[i])),
 * ctx_dev and gate_dev [S][H*hd] on the handle's device */
int moty_cuda_attn_gate_dev(MotyCudaAttn *a, float *ctx_dev, const float *gate_dev, int S, void *stream);

/* ---- load-time quantizers (weights) -----------------------------------------
 * moty_quantize_rows (nn/quant.c:12-33) with bits = 8: w [O][I] f32 host ->
 * q [O][I] int8, scale [O] f32 host, computed on the GPU. */
int moty_cuda_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I);
/* moty_pack_q4r4_block over a whole matrix (nn/quant.c:157-179,
 * runtime/rt_model_load.h:85-121): q4 [ceil(O/4)][I/32][64], s16 [..][4]. */
int moty_cuda_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16);

#ifdef __cplusplus
}
#endif
#endif /* MOTY_CUDA_H */
