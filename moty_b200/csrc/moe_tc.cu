// moe_tc.cu -- the grouped expert products of a routed int8 MoE batch on the 5th-generation tensor cores.
//
// Replaces the three moty_matmul_q_s calls per expert of moe_batch_core (nn/moe.c:186-199) and the SiLU between them
// for batches (prefill): the routed rows are gathered per expert (pair order: by expert, then by token), and
//   pass 1  for every (expert, tile of BN routed rows, 128 rows of the expert's FFN width):
//             gate and up products of those rows in ONE work item -- two tcgen05 accumulators in TMEM fed by the
//             same activation tile -- and in the epilogue (scale*sx)*acc for both, silu(g)*u, one f32 store:
//             h[pair][i]; no [P][I] gate/up buffers, no activation kernel, no memsets;
//   pass 2  h rows re-quantized per row (nn/moe.c:117-124, the ordinary row quantizer), then the down product with
//           the expert's [D][I] matrix, epilogue (ds*hs)*acc -> hout[pair][d]; the ordered combine follows.
// The kernel is the persistent TMA + tcgen05 pipeline of gemm_q8_tc.cu (warp 0 producer, warp 1 issuer, eight
// epilogue warps, two TMEM buffers, bounded waits) with a WORK LIST instead of a dense tile grid: the routing plan
// writes one entry per (expert, row tile) on the device and its count; work item = entry x 128-row block.  The
// experts of a layer live in one slab [E_local][rows][cols], so a single tensor map over the slab serves every
// expert (row coordinate = expert * rows + block).  A tile that runs past its expert's rows or past its routed rows
// computes on whatever follows and the epilogue drops those rows and columns.
// Integer accumulation is exact and the f32 steps are the reference's, so the results carry the same bits as the
// mma.sync path it replaces and as the CPU reference.
#include "tc_common.cuh"
#include "moe.cuh"

namespace {

constexpr int MT_EPI_WARPS = 8, MT_THREADS = 64 + 32 * MT_EPI_WARPS;

struct MoeTcArgs {
    const Q8Tile *tiles;            // [ntiles]: w = the expert's matrix of this pass (gate or down), scale = its row scales
    const Q8Tile *tiles2;           // pass 1: the same tiles for the up matrices (scale pointers); null in pass 2
    const int *ntiles_dev;
    const int8_t *slab;             // base of the matrices the tiles' w pointers point into
    size_t expert_bytes;            // bytes per expert in that slab
    const float *sx;                // [P] activation scale per routed row
    float *out;                     // pass 1: h [P][M]; pass 2: hout [P][M]
    int M;                          // rows per expert of this pass: I (pass 1) or D (pass 2)
    int Kdim;                       // row length in bytes: D (pass 1) or I (pass 2)
    int *err;
};

// GATEUP: pass 1 (two A tiles per stage, two accumulators per buffer, SiLU epilogue)
template <int BN, int STAGES, bool GATEUP>
__global__ void __launch_bounds__(MT_THREADS, 1) moe_tc_kernel(const __grid_constant__ CUtensorMap mapA,
                                                               const __grid_constant__ CUtensorMap mapA2,
                                                               const __grid_constant__ CUtensorMap mapB, MoeTcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int NA = GATEUP ? 2 : 1;
    constexpr int A_BYTES = NA * BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int NBUF = 2;
    constexpr uint32_t TMEM_COLS = NBUF * NA * BN < 32 ? 32 : NBUF * NA * BN;
    static_assert(NBUF * NA * BN <= 512, "TMEM holds 512 columns");
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (a.Kdim + BKB - 1) / BKB;
    const int ntm = (a.M + BM - 1) / BM;

    pdl_trigger();                                   // barriers and TMEM are set up under the previous kernel's tail
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int i = 0; i < STAGES; i++) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&tmem_full_bar[i], 1); mbar_init(&tmem_empty_bar[i], MT_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    volatile int *abort_flag = &abort_s;
    pdl_wait();                                      // the plan, the gathered codes and their scales come from earlier launches
    const int nitems = *a.ntiles_dev * ntm;          // written by the plan kernel earlier on this stream

    // item -> (row tile entry, 128-row block of the expert); consecutive items share the entry, so CTAs running side by
    // side read the same activation tile (second fetch from L2) against different weight blocks
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = blockIdx.x; t < nitems; t += gridDim.x) {
                const int te = t / ntm, mb = t - te * ntm;
                const Q8Tile tl = a.tiles[te];
                const int le = (int)((size_t)(tl.w - a.slab) / a.expert_bytes);
                const int arow = le * a.M + mb * BM, brow = tl.row0;
                bool ok = true;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int st = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&empty_bar[st], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&full_bar[st], STAGE_BYTES);
                    uint8_t *sa = smem + (size_t)st * STAGE_BYTES;
                    tma_load_2d(sa, &mapA, kb * BKB, arow, &full_bar[st]);
                    if (GATEUP) tma_load_2d(sa + BM * BKB, &mapA2, kb * BKB, arow, &full_bar[st]);
                    tma_load_2d(sa + A_BYTES, &mapB, kb * BKB, brow, &full_bar[st]);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, tl = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < nitems && ok; t += gridDim.x, tl++) {
                const uint32_t buf = tl % NBUF, use = tl / NBUF;
                ok = mbar_wait(&tmem_empty_bar[buf], (use & 1) ^ 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem_base + buf * NA * BN;
                for (int kb = 0; kb < nkb; kb++, it++) {
                    const int st = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&full_bar[st], ph, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_u32(smem + (size_t)st * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < BKB / 32; k4++) {
                        if (kb * BKB + k4 * 32 >= a.Kdim) break;                  // nothing but zero fill beyond the row
                        umma_i8(tacc, umma_desc(sa + k4 * 32), umma_desc(sb + k4 * 32), idesc, (kb | k4) != 0);
                        if (GATEUP)
                            umma_i8(tacc + BN, umma_desc(sa + BM * BKB + k4 * 32), umma_desc(sb + k4 * 32), idesc, (kb | k4) != 0);
                    }
                    umma_commit(&empty_bar[st]);
                }
                if (ok) umma_commit(&tmem_full_bar[buf]);
            }
        }
    } else {
        const int q = warp & 3, half = (warp - 2) >> 2;
        constexpr int CPW = BN >= 32 ? BN / 2 : BN;
        const int col_lo = BN >= 32 ? half * CPW : 0;
        const bool works = BN >= 32 || half == 0;
        uint32_t tl = 0;
        for (int t = blockIdx.x; t < nitems; t += gridDim.x, tl++) {
            const int te = t / ntm, mb = t - te * ntm;
            const uint32_t buf = tl % NBUF, use = tl / NBUF;
            int ok = lane == 0 ? (int)mbar_wait(&tmem_full_bar[buf], use & 1, abort_flag) : 1;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (works) {
                const Q8Tile tile = a.tiles[te];
                const int i = mb * BM + q * 32 + lane;                          // row of the expert's matrix
                const bool row_ok = i < a.M;
                const float sc = row_ok ? __ldg(tile.scale + i) : 0.f;
                float sc2 = 0.f;
                if (GATEUP) sc2 = row_ok ? __ldg(a.tiles2[te].scale + i) : 0.f;
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_lo + CPW; c0 += 16) {
                    if (c0 >= tile.nrows) break;                                // warp-uniform: routed rows of this tile
                    uint32_t r[16], r2[16];
                    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * NA * BN + (uint32_t)c0;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                        : "r"(taddr));
                    if (GATEUP)
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                            : "=r"(r2[0]), "=r"(r2[1]), "=r"(r2[2]), "=r"(r2[3]), "=r"(r2[4]), "=r"(r2[5]), "=r"(r2[6]), "=r"(r2[7]),
                              "=r"(r2[8]), "=r"(r2[9]), "=r"(r2[10]), "=r"(r2[11]), "=r"(r2[12]), "=r"(r2[13]), "=r"(r2[14]), "=r"(r2[15])
                            : "r"(taddr + BN));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int c = c0 + j;
                            if (c < tile.nrows) {
                                const int p = tile.row0 + c;
                                const float sx = __ldg(a.sx + p);
                                // (scale[i] * sx) * (float)dot, left to right (nn/matmul.c:34)
                                float v = __fmul_rn(__fmul_rn(sc, sx), (float)(int)r[j]);
                                if (GATEUP) v = moty_silu_mul(v, __fmul_rn(__fmul_rn(sc2, sx), (float)(int)r2[j]));   // nn/moe.c:197
                                a.out[(size_t)p * a.M + i] = v;
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty_bar[buf])) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_s) {
        for (int i = 0; i < 1000; i++) __nanosleep(1000);       // copies that may still be in flight land before the CTA's memory goes
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_s) atomicExch(a.err, 1);
}

template <int BN, int STAGES, bool GATEUP>
int launch_moe_tc_t(const MoeTcArgs &a, const void *slab, const void *slab2, int slab_rows, const int8_t *b, int brows,
                    int sms, cudaStream_t st) {
    CUtensorMap mapA, mapA2, mapB;
    CKR(make_map(&mapA, slab, slab_rows, a.Kdim, BM));
    CKR(make_map(&mapA2, GATEUP ? slab2 : slab, slab_rows, a.Kdim, BM));
    CKR(make_map(&mapB, b, brows, a.Kdim, BN));
    constexpr int NA = GATEUP ? 2 : 1;
    size_t smem = (size_t)STAGES * (NA * BM * BKB + BN * BKB) + 1024;
    auto k = moe_tc_kernel<BN, STAGES, GATEUP>;
    CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(moty_launch_pdl(k, dim3(sms), dim3(MT_THREADS), smem, st, mapA, mapA2, mapB, a));
    return 0;
}

}  // namespace

// rows per tile the plan must cut the experts' routed rows into for this path: 16, 32, 64 or 128 -- about the
// average rows per expert.  (Tiles of twice that, so that most experts stream their matrices once, measured slower
// on the OLMoE layer at 512 tokens: 217 against 197 us -- fewer, longer work items balance worse over 148 SMs.)
int moe_tc_tile_rows(long long rows_per_expert) {
    return rows_per_expert >= 96 ? 128 : (rows_per_expert >= 40 ? 64 : (rows_per_expert >= 20 ? 32 : 16));
}

// 128-byte swizzled tiles want 16-byte row strides; rows shorter than a K block gain nothing
bool moe_tc_supported(int I, int D) { return I % 16 == 0 && D % 16 == 0 && I >= 128 && D >= 128; }

// pass 1: h[p][i] = silu(gate) * up for every routed row p (pair order), i < I.  xg [P][D]: the routed rows' codes
// gathered in pair order, sxg [P] their scales.  g_slab/u_slab: [E_local][I][D].
int launch_moe_tc_gateup(const Q8Tile *t_gate, const Q8Tile *t_up, const int *ntiles_dev, int tile_rows,
                         const int8_t *g_slab, const int8_t *u_slab, int E_local, const int8_t *xg, const float *sxg,
                         int P, float *h, int I, int D, int *err, int sms, cudaStream_t st) {
    MoeTcArgs a;
    a.tiles = t_gate; a.tiles2 = t_up; a.ntiles_dev = ntiles_dev; a.slab = g_slab; a.expert_bytes = (size_t)I * D;
    a.sx = sxg; a.out = h; a.M = I; a.Kdim = D; a.err = err;
    switch (tile_rows) {
    case 16: return launch_moe_tc_t<16, 4, true>(a, g_slab, u_slab, E_local * I, xg, P, sms, st);
    case 32: return launch_moe_tc_t<32, 4, true>(a, g_slab, u_slab, E_local * I, xg, P, sms, st);
    case 64: return launch_moe_tc_t<64, 4, true>(a, g_slab, u_slab, E_local * I, xg, P, sms, st);
    case 128: return launch_moe_tc_t<128, 4, true>(a, g_slab, u_slab, E_local * I, xg, P, sms, st);
    }
    return moty_set_error(MOTY_CUDA_EARG, "moe_tc: tile of %d rows", tile_rows);
}

// pass 2: hout[p][d] = (ds[d] * hs[p]) * dot(down[d], hq[p]).  d_slab: [E_local][D][I].
int launch_moe_tc_down(const Q8Tile *t_down, const int *ntiles_dev, int tile_rows, const int8_t *d_slab, int E_local,
                       const int8_t *hq, const float *hs, int P, float *hout, int I, int D, int *err, int sms, cudaStream_t st) {
    MoeTcArgs a;
    a.tiles = t_down; a.tiles2 = nullptr; a.ntiles_dev = ntiles_dev; a.slab = d_slab; a.expert_bytes = (size_t)I * D;
    a.sx = hs; a.out = hout; a.M = D; a.Kdim = I; a.err = err;
    switch (tile_rows) {
    case 16: return launch_moe_tc_t<16, 6, false>(a, d_slab, nullptr, E_local * D, hq, P, sms, st);
    case 32: return launch_moe_tc_t<32, 6, false>(a, d_slab, nullptr, E_local * D, hq, P, sms, st);
    case 64: return launch_moe_tc_t<64, 6, false>(a, d_slab, nullptr, E_local * D, hq, P, sms, st);
    case 128: return launch_moe_tc_t<128, 6, false>(a, d_slab, nullptr, E_local * D, hq, P, sms, st);
    }
    return moty_set_error(MOTY_CUDA_EARG, "moe_tc: tile of %d rows", tile_rows);
}
