// moe.cuh -- argument blocks shared by moe.cu and the C-ABI layer.
#pragma once
#include "kernels.cuh"

struct MoePlanArgs {
    const int *idx;            // [S][K] routed expert ids
    int S, K, E, e_lo, e_hi;
    int T;                     // rows per tile (8 for int8 experts, 4 for Q4R4)
    int order;                 // 0 selection order, 1 ascending expert id
    int q8;                    // 1 int8 experts, 0 Q4R4 experts
    // expert slabs: expert e (local index e - e_lo) starts at base + local * stride
    const int8_t *g8, *u8, *d8; const float *gs, *us, *ds;
    const uint8_t *g4, *u4, *d4; const uint16_t *gs16, *us16, *ds16;
    size_t gstride, gsstride, dstride, dsstride;   // in elements of the respective arrays
    // outputs
    int *pair_tok, *pos_of, *ord, *ntiles, *npairs;
    uint8_t *form;             // Q4R4 only, else null
    Q8Tile *t8_gate, *t8_up, *t8_down;
    Q4Tile *t4_gate, *t4_up, *t4_down;
};

int launch_moe_plan(const MoePlanArgs &a, cudaStream_t st);
int launch_moe_combine(float *out, const float *h, const float *w, const int *pos_of, const int *ord,
                       int S, int K, int D, cudaStream_t st);
int launch_moe_combine_sk(float *out, const float *h, const float *w, const int *idx,
                          int S, int K, int D, int order, cudaStream_t st);
int launch_f32_rows(const float *W, const float *x, float *y, int S, int I, int O, cudaStream_t st);

// ---- moe_decode.cu: one routed token through int8 experts in two streaming kernels ----
bool moe_decode_q8_supported(int K, int I, int D);
int launch_moe_decode_q8(const int *idx, const float *w, const int8_t *g, const int8_t *u, const int8_t *d,
                         const float *gs, const float *us, const float *ds, size_t gstride, size_t gsstride,
                         size_t dstride, size_t dsstride, const float *x, float *h, float *out,
                         int K, int I, int D, int e_lo, int e_hi, int sms, cudaStream_t st,
                         const float *logits = nullptr, int E = 0, int norm_topk = 0);   // logits given (E <= 2048): the first
                                                                                         // kernel routes the token itself and
                                                                                         // leaves the selections in idx / w

// ---- moe_decode_q4.cu: the same for Q4R4 experts ----
bool moe_decode_q4_supported(int K, int I, int D);
int launch_moe_decode_q4(const int *idx, const float *w, const uint8_t *g, const uint8_t *u, const uint8_t *d,
                         const uint16_t *gs, const uint16_t *us, const uint16_t *ds, size_t gstride, size_t gsstride,
                         size_t dstride, size_t dsstride, const float *x, float *h, float *out,
                         int K, int I, int D, int e_lo, int e_hi, int sms, cudaStream_t st);

// ---- moe_decode_fused.cu: router + gate/up + down of one token in one cooperative launch ----
bool moe_decode_fused_q8_supported(int E, int K, int I, int D);
int launch_moe_decode_fused_q8(const float *logits, int E, int norm_topk, int *idx_out, float *w_out,
                               const int8_t *g, const int8_t *u, const int8_t *d, const float *gs, const float *us,
                               const float *ds, size_t gstride, size_t gsstride, size_t dstride, size_t dsstride,
                               const float *x, float *h, float *out, float *rows, int K, int I, int D, int e_lo, int e_hi,
                               unsigned *bar, int *err, int sms, cudaStream_t st, float *const *rows_peer = nullptr, int npeer = 0);

// ---- moe_decode_fused_q4.cu: the same for Q4R4 experts ----
bool moe_decode_fused_q4_supported(int E, int K, int I, int D);
int launch_moe_decode_fused_q4(const float *logits, int E, int norm_topk, int *idx_out, float *w_out,
                               const uint8_t *g, const uint8_t *u, const uint8_t *d, const uint16_t *gs,
                               const uint16_t *us, const uint16_t *ds, size_t gstride, size_t gsstride,
                               size_t dstride, size_t dsstride, const float *x, int8_t *hq, float *hs, int *hsum,
                               float *out, float *rows, int K, int I, int D, int e_lo, int e_hi, unsigned *bar, int *err,
                               int sms, cudaStream_t st, float *const *rows_peer = nullptr, int npeer = 0, int chained = 0);

// ---- moe_tc.cu: the grouped expert products of an int8 batch on tcgen05 (work list = plan tiles x 128-row blocks) ----
bool moe_tc_supported(int I, int D);
int moe_tc_tile_rows(long long rows_per_expert);
int launch_moe_tc_gateup(const Q8Tile *t_gate, const Q8Tile *t_up, const int *ntiles_dev, int tile_rows,
                         const int8_t *g_slab, const int8_t *u_slab, int E_local, const int8_t *xg, const float *sxg,
                         int P, float *h, int I, int D, int *err, int sms, cudaStream_t st);
int launch_moe_tc_down(const Q8Tile *t_down, const int *ntiles_dev, int tile_rows, const int8_t *d_slab, int E_local,
                       const int8_t *hq, const float *hs, int P, float *hout, int I, int D, int *err, int sms, cudaStream_t st);

// ---- moe.cu: the exchange step of the expert-parallel decode over peer memory ----
int launch_moe_peer_combine(float *out, const float *table, const float *w, const int *idx, int K, int D,
                            unsigned *const *flags_peer, unsigned *flags_local, int world, int rank, unsigned epoch,
                            int *err, cudaStream_t st);
