// kernels.cuh -- launchers of the device kernels (all enqueue on `st`, none synchronise).
#pragma once
#include "common.cuh"
#include "waits.cuh"

// ---- quant.cu ---------------------------------------------------------------
int launch_qrow_i8_scatter(const float *x, const int *pos_of, int S, int K, int8_t *xg, float *sxg, int n, cudaStream_t st);
int launch_qrow_i8_counted(const float *x, int8_t *q, float *scale, int rows_max, int n, const int *nrows_dev, cudaStream_t st);
int launch_qrow_i8(const float *x, int8_t *q, float *scale, int rows, int n, cudaStream_t st);
int launch_quant_g32(const float *x, int rows, int I, int8_t *xq, float *xs, int32_t *xsum, cudaStream_t st);
int launch_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I, cudaStream_t st);
int launch_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16, cudaStream_t st);

// ---- gemv_q8.cu ---------------------------------------------------------------
// One Q8_0 product over pre-quantized activation rows:
//   y[yrow(t)][o] = (scale[o] * sx[xrow(t)]) * (float)dot(W[o], xi[xrow(t)])
// A "tile" is up to 8 activation rows that share one weight matrix.  The dense
// drivers use identity row maps and a single matrix; the MoE block passes a tile
// table so that every tile can point at another expert's matrix.
struct Q8Tile {
    const int8_t *w;        // [O][I]
    const float *scale;     // [O]
    int row0;               // first entry of xmap/ymap (or first row when maps are null)
    int nrows;              // 1..8
};
struct Q8Args {
    const int8_t *w; const float *scale;        // dense: the one matrix
    const Q8Tile *tiles; const int *ntiles_dev;  // grouped: tile table (+ device count), else null
    int ntiles_max;
    const int8_t *xi; const float *sx;          // quantized activation rows [..][I], scales
    const int *xmap, *ymap;                     // optional gather / scatter row maps
    float *y; int ldy;                          // output rows, leading dimension
    int32_t *acc;                               // optional int32 accumulators, same indexing as y
    int S, I, O;
};
int launch_q8_small(const Q8Args &a, int sms, cudaStream_t st);
int launch_dot_i8i8_rows(const int8_t *w, const int8_t *x, int nrows, int n, int32_t *out, cudaStream_t st);
int launch_dot_i4i8_rows(const uint8_t *w4, const int8_t *x, int nrows, int n, int32_t *out, cudaStream_t st);

int launch_q8_any(const int8_t *W, const float *scale, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                  int S, int I, int O, cudaStream_t st);
int gemv_q8_init_device();

// ---- gemv_q8_stream.cu -------------------------------------------------------
// persistent streaming GEMV for 1..8 rows; S == 1 quantizes x (f32) in the kernel
int launch_q8_stream(const int8_t *w, const float *scale, const float *x, const int8_t *xi, const float *sx,
                     float *y, int32_t *acc, int S, int I, int O, int *counters, unsigned long long *cell,
                     int sms, cudaStream_t st, const float *t = nullptr, const float *g = nullptr, float *xout = nullptr,
                     float eps = 0.f, const float *gt = nullptr);
                                         // t (S == 1, I <= 4096): the row is rmsnorm(x + t) * g, and x + t goes to xout;
                                         // with gt the sum is x + rmsnorm(t) * gt (resnorm.cuh)
int q4r4_init_device();

// ---- gemm_q8_tc.cu --------------------------------------------------------------
// tcgen05 int8 GEMM for S >= 16: weights through a TMA descriptor, int32
// accumulators in TMEM, epilogue (scale[o]*sx[s])*(float)acc.
bool q8_tc_supported(int S, int I, int O);
int q8_tc_make_tmap(MotyCudaMat *m);
int launch_q8_tc(const MotyCudaMat *w, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                 int S, DevCtx *c, cudaStream_t st);

// ---- q4r4.cu ----------------------------------------------------------------------
struct Q4Tile { const uint8_t *w; const uint16_t *d; int row0; int nrows; };
struct Q4Args {
    const uint8_t *w; const uint16_t *d;
    const Q4Tile *tiles; const int *ntiles_dev; int ntiles_max;
    const int8_t *xq; const float *xs; const int32_t *xsum;   // group-quantized rows
    const int *xmap, *ymap;
    const uint8_t *form;     // per activation row: 1 = 4-token-tile formula, 0 = token-by-token
    float *y; int ldy;
    int S, I, O;
};
int launch_q4r4_small(const Q4Args &a, int sms, cudaStream_t st);
// which of the reference's two kernels each of S tokens goes through
int launch_q4r4_forms(uint8_t *form, int S, cudaStream_t st);

// ---- q4r4_gemv1.cu: Q4R4 decode GEMV for matrices with many rows (lane = row) ----
bool q4r4_gemv1_supported(int I, int O, int sms);
int launch_q4r4_gemv1(const uint8_t *w, const uint16_t *d, const float *x, float *y, int I, int O, int sms, cudaStream_t st);

// ---- norm.cu: RMS norm of rows, residual add, int8 embedding rows ----
int launch_rmsnorm_rows(float *out, const float *x, const float *w, int S, int D, float eps, cudaStream_t st);
int launch_add(float *y, const float *x, long long n, cudaStream_t st);
int launch_add_rmsnorm_rows(float *x, const float *t, float *out, const float *w, int S, int D, float eps, cudaStream_t st);
// x += rmsnorm(t) * g1, then (out given) out = rmsnorm(x) * g2
int launch_normadd_rmsnorm_rows(float *x, const float *t, const float *g1, float *out, const float *g2, int S, int D, float eps,
                                cudaStream_t st);
int launch_embed_rows(float *dst, const int8_t *q, const float *qs, const int *ids, int S, int D, int V, float scale, cudaStream_t st);

// ---- attn.cu: attention core between the projections (QK-norm + RoPE, KV store, scores, softmax, accumulation) ----
int launch_attn_core(float *ctx, float *q, float *k, const float *v, int S, int pos_base, int H, int KV, int hd, int rot,
                     float theta, float eps, const float *qn, const float *kn, float *K, float *V, int8_t *K8, int8_t *V8,
                     float *Ks, float *Vs, int max_t, float *part, const int *pos_dev, int *err, int sms, cudaStream_t st,
                     int gemma = 0, int window = 0, float scale = 0.f, const float *vn = nullptr);
size_t attn_scratch_bytes(int S, int H, int KV, int hd, int sms);
int launch_attn_gate(float *ctx, const float *gate, long long n, cudaStream_t st);

// ---- q4r4_gemv2.cu: Q4R4 / Q8R4 decode GEMV in two phases (parallel integer sums, then the chain) ----
bool q4r4_gemv2_supported(int I, int O, int q8, int sms);
size_t q4r4_gemv2_scratch_bytes(int I, int O);
int launch_q4r4_gemv2(const uint8_t *w, const uint16_t *d, const float *x, float *y, float *ab, int *err,
                      int I, int O, int q8, int sms, cudaStream_t st);

// the reference's default (IDOT4 unset) product for the same layout: f32 activations x dequantized int4
// ---- i4g_mma.cu: WF_I4G (grouped int4, group 32, f32 group scales) x row-quantized activations, two rows and more:
// one integer MMA per group, the f32 chain in registers; i4g.cu: the reference's default f32 x int4 product ----
size_t i4g_mma_scratch_bytes(int S, int I);
int launch_i4g_mma(const uint8_t *w4, const float *scale, const int8_t *xi, const float *sx, int *rec, float *y,
                   int S, int I, int O, int sms, cudaStream_t st);
int launch_i4g_f32_rows(const uint8_t *w4, const float *scale, const float *x, float *y, int S, int I, int O, cudaStream_t st);
int launch_i4g_gemv2(const uint8_t *w4, const float *gscale, const int8_t *xi, const float *sx, float *y, float *ab,
                     int *err, int I, int O, int sms, cudaStream_t st);

// ---- q4r4_gemv_bulk.cu: Q4R4 decode GEMV for few long rows (lane = row, fed by bulk async copies) ----
bool q4r4_gemv_bulk_supported(int I, int O, int sms);
int launch_q4r4_gemv_bulk(const uint8_t *w, const uint16_t *d, const int8_t *xq, const float *xs, const int32_t *xsum,
                          float *y, int I, int O, int *err, int sms, cudaStream_t st);

// ---- q8_mma.cu: Q8_0 x a small batch (mma.sync, weights streamed once), dense and grouped ----
bool q8_mma_supported(int S, int I, int O);
int q8_mma_ksplit(int S, int I, int O, int sms);
size_t q8_mma_scratch_bytes(int S, int O);
int launch_q8_mma(const int8_t *w, const float *scale, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                  int S, int I, int O, void *scratch, int sms, cudaStream_t st);
int launch_q8_mma_grouped(const Q8Tile *tiles, const int *ntiles_dev, int ntiles_max, int tile_rows,
                          const int8_t *xi, const float *sx, const int *xmap, float *y, int ldy, int I, int O,
                          cudaStream_t st);

// ---- q4r4_mma.cu: Q4R4 x a batch of rows, integer MMA per group + the sequential f32 chain ----
int launch_q4r4_mma(const uint8_t *w, const uint16_t *d, const int8_t *xq, const float *xs, const int32_t *xsum,
                    int4 *rec, float *y, int ldy, int S, int I, int O, int q8, int sms, cudaStream_t st, int relax = 0);

int launch_q4r4_mma_grouped(const Q4Tile *tiles, const int *ntiles_dev, int ntiles_max, int tile_rows,
                            const int *npairs_dev, const int8_t *xq, const float *xs, const int32_t *xsum,
                            const int *xmap, const uint8_t *form, int4 *rec, int build_rec, float *y, int ldy, int P,
                            int I, int O, cudaStream_t st, int relax = 0, int sms = 148);

// ---- router.cu ----------------------------------------------------------------------
int launch_route(const float *logits, int rows, int E, int K, int *idx, float *w, float *probs,
                 int do_softmax, int norm_topk, cudaStream_t st, const float *bias = nullptr);
int launch_argmax_scratch(const float *v, int n, int *out, float *pv, int *pi, cudaStream_t st);

// ---- moe.cu / ffn -------------------------------------------------------------------
int launch_act_mul(float *g, const float *u, int64_t n, int act, cudaStream_t st);

// ---- q4r4_stream.cu -------------------------------------------------------------------
// persistent Q4R4 GEMV for 1..4 rows; S == 1 with x != null quantizes the row in the kernel
int launch_q4r4_stream(const uint8_t *w, const uint16_t *d, const float *x, const int8_t *xq, const float *xs,
                       const int32_t *xsum, const uint8_t *form, float *y, int S, int I, int O, int sms, cudaStream_t st);

// ---- selftest.cu: the give-up path of the bounded waits, run on purpose with a short limit ----
int launch_selftest_expire(int which, int *err_dev, unsigned *gridbar_words, cudaStream_t st);

// per-row int4 rows -> int8 codes (nibble - 8), quant.cu
int launch_i4_rows_to_i8(const uint8_t *q4, int8_t *q8, long long rows, int n, cudaStream_t st);

// ---- hostio.cu: activations in / results out between mapped (pinned) host buffers and the device, by kernels ----
int launch_stage_in(float *dst, const float *src_host, long long n, cudaStream_t st);
int launch_tail_out(float *dst_host, const float *src, long long n, unsigned *ctr, unsigned *flag_host, int sms, cudaStream_t st);

// ---- gemv_q8_gateup.cu: h = act(gate . x) * (up . x) for one token in one launch (rows of at most 4096 values) ----
bool q8_gateup_supported(int I, int D);
int launch_q8_gateup(const int8_t *g, const float *gs, const int8_t *u, const float *us, const float *x, float *h, int I, int D,
                     int act, int sms, cudaStream_t st, const float *t = nullptr, const float *g_t = nullptr,
                     const float *g_x = nullptr, float *xout = nullptr, float eps = 0.f);
                                         // t: the activation row is rmsnorm(x + t) * g_x (g_t: x + rmsnorm(t) * g_t), the sum goes to xout

// ---- gemv_q8_multi.cu: up to eight independent S = 1 Q8_0 products in one launch ----
bool q8_multi_supported(int I);
int launch_q8_multi(int n, const int8_t *const *w, const float *const *scale, const float *const *x, float *const *y,
                    const int *O, const int *I, int sms, cudaStream_t st, unsigned long long *const *cells = nullptr);
