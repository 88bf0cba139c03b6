// gemm_q8_tc.cu -- Q8_0 prefill GEMM on the 5th-generation tensor cores.
//
//   acc[o][s] = sum_i W[o][i] * xi[s][i]       int8 x int8 -> int32, exact
//   y[s][o]   = (scale[o] * sx[s]) * (float)acc (nn/matmul.c:29-36)
//
// Persistent CTAs (one per SM) walk over 128 (output rows) x BN (tokens) tiles:
//   warp 0   producer: TMA loads of the W tile [128 x 128 B] and the activation
//            tile [BN x 128 B] into a STAGES-deep shared-memory ring, 128-byte swizzle,
//            completion on mbarriers (per-CTA loads only, no multicast);
//   warp 1   issues tcgen05.mma.cta_group::1.kind::i8 (M=128, N=BN, K=32; four per
//            128-byte K block) accumulating int32 in one of two TMEM accumulators,
//            tcgen05.commit frees the ring slots and finally signals the epilogue;
//   warps 2-5 epilogue: tcgen05.ld of their 32-lane TMEM quarter, scale, coalesced
//            stores of y (32 consecutive output rows per instruction), overlapped with
//            the MMAs of the next tile through the second accumulator.
// W is the A operand so that M = 128 weight rows fill the tensor-core datapath even
// when only 16 tokens are present; the kernel is then HBM-bound on the weights.
//
// Every mbarrier wait is bounded: on expiry the waiter raises a CTA-wide abort
// flag and a device error word, all roles fall through to the common exit, the
// TMEM columns are freed, and the host reports MOTY_CUDA_EKERNEL.
#include "tc_common.cuh"

namespace {

// warp 0: TMA producer; warp 1: MMA issuer; warps 2..9: epilogue (two warps per TMEM lane quarter, each
// taking half of the accumulator's columns)
constexpr int TC_EPI_WARPS = 8, TC_THREADS = 64 + 32 * TC_EPI_WARPS;

struct TcArgs {
    const float *scale; const float *sx; float *y; int32_t *acc;
    int S, I, O;
    int *err;
    // split over K (matrices with few 128-row tiles): work item = (tile, split); every split leaves its
    // exact int32 partial sums in part[split][S][O] and tc_splitk_finish_kernel adds and scales them
    int ksplit; int32_t *part;
};

template <int BN, int STAGES, int MT>
__global__ void __launch_bounds__(TC_THREADS, 1) q8_tc_kernel(const __grid_constant__ CUtensorMap mapA,
                                                       const __grid_constant__ CUtensorMap mapB, TcArgs a) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment for the swizzled tiles
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    // MT = 2: two 128-row weight sub-tiles share one activation tile (half the activation bytes per
    // MAC through shared memory); their two accumulators fill TMEM, so no double buffering then
    constexpr int A_BYTES = MT * BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int NBUF = (2 * MT * BN <= 512) ? 2 : 1;
    __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], tmem_full_bar[2], tmem_empty_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (a.I + BKB - 1) / BKB;
    const int ntn = (a.S + BN - 1) / BN, ntm = (a.O + MT * BM - 1) / (MT * BM);
    const int KS = a.ksplit, nks = (nkb + KS - 1) / KS;                 // K blocks per split (the last may hold fewer, never none)
    const int ntiles = ntm * ntn * KS;                                   // work items; item = tile * KS + split
    const int krot = (int)((blockIdx.x * 5u) % (unsigned)nks);
    // two accumulators of BN columns: the epilogue of one tile overlaps the MMAs of the next
    constexpr uint32_t TMEM_COLS = NBUF * MT * BN < 32 ? 32 : NBUF * MT * BN;

    pdl_trigger();                                                       // barriers and TMEM are set up under the previous kernel's tail
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int i = 0; i < STAGES; i++) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < 2; i++) { mbar_init(&tmem_full_bar[i], 1); mbar_init(&tmem_empty_bar[i], TC_EPI_WARPS); }
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
    pdl_wait();                                                          // activation codes and scales come from the quantizer launch

    // Persistent over output tiles.  Consecutive tile numbers share the weight rows (same m,
    // next n), so CTAs running side by side fetch the same W tile and the second fetch hits L2.
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;                                         // ring position, continuous across tiles
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x) {
                const int tile = t / KS, ks = t - tile * KS;
                const int m0 = (tile / ntn) * MT * BM, n0 = (tile % ntn) * BN;
                const int kb_lo = ks * nks, nk = nkb - kb_lo < nks ? nkb - kb_lo : nks;
                bool ok = true;
                for (int kb = 0; kb < nk; kb++, it++) {
                    const int st = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&empty_bar[st], ph ^ 1, abort_flag);
                    if (!ok) break;
                    mbar_expect_tx(&full_bar[st], STAGE_BYTES);
                    uint8_t *sa = smem + (size_t)st * STAGE_BYTES;
                    // every CTA starts its K loop at another block: integer accumulation is order
                    // independent, and the CTAs stop hammering the same activation tile in L2 together
                    const int kr = kb_lo + (kb + krot) % nk;
                    tma_load_2d(sa, &mapA, kr * BKB, m0, &full_bar[st]);
                    if (MT == 2) tma_load_2d(sa + BM * BKB, &mapA, kr * BKB, m0 + BM, &full_bar[st]);
                    tma_load_2d(sa + A_BYTES, &mapB, kr * BKB, n0, &full_bar[st]);
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D = s32, A = B = signed int8, both K-major, N = BN, M = 128
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            uint32_t it = 0, tl = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < ntiles && ok; t += gridDim.x, tl++) {
                const uint32_t buf = tl % NBUF, use = tl / NBUF;
                ok = mbar_wait(&tmem_empty_bar[buf], (use & 1) ^ 1, abort_flag);   // epilogue has drained this accumulator
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tacc = tmem_base + buf * MT * BN;
                const int ks = t % KS, kb_lo = ks * nks, nk = nkb - kb_lo < nks ? nkb - kb_lo : nks;
                for (int kb = 0; kb < nk; kb++, it++) {
                    const int st = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    ok = mbar_wait(&full_bar[st], ph, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t sa = smem_u32(smem + (size_t)st * STAGE_BYTES);
                    const uint32_t sb = sa + A_BYTES;
#pragma unroll
                    for (int k4 = 0; k4 < BKB / 32; k4++) {
                        if ((kb_lo + (kb + krot) % nk) * BKB + k4 * 32 >= a.I) break;   // nothing but zero fill beyond I
                        umma_i8(tacc, umma_desc(sa + k4 * 32), umma_desc(sb + k4 * 32), idesc, (kb | k4) != 0);
                        if (MT == 2)
                            umma_i8(tacc + BN, umma_desc(sa + BM * BKB + k4 * 32), umma_desc(sb + k4 * 32), idesc, (kb | k4) != 0);
                    }
                    umma_commit(&empty_bar[st]);                           // slot reusable when these MMAs retire
                }
                if (ok) umma_commit(&tmem_full_bar[buf]);                  // accumulator complete
            }
        }
    } else {
        // epilogue: warp w may touch TMEM lanes 32*(w%4) .. +31; the two warps of a quarter split the columns
        const int q = warp & 3, half = (warp - 2) >> 2;
        constexpr int CPW = BN >= 32 ? BN / 2 : BN;                       // columns per warp (BN = 16: the second warp idles)
        const int col_lo = BN >= 32 ? half * CPW : 0;
        const bool works = BN >= 32 || half == 0;
        uint32_t tl = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, tl++) {
            const int tile = t / KS, ks = t - tile * KS;
            const int m0 = (tile / ntn) * MT * BM, n0 = (tile % ntn) * BN;
            const uint32_t buf = tl % NBUF, use = tl / NBUF;
            // one lane waits, the warp follows its verdict (tcgen05.ld is warp-collective)
            int ok = lane == 0 ? (int)mbar_wait(&tmem_full_bar[buf], use & 1, abort_flag) : 1;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int mt = 0; mt < MT && works; mt++) {
                const int o = m0 + mt * BM + q * 32 + lane;
                const bool row_ok = o < a.O;
                const float sc = row_ok ? __ldg(a.scale + o) : 0.f;
#pragma unroll 1
                for (int c0 = col_lo; c0 < col_lo + CPW; c0 += 16) {
                    const int s0 = n0 + c0;
                    if (s0 >= a.S) break;                                  // warp-uniform
                    uint32_t r[16];
                    uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (buf * MT + mt) * BN + (uint32_t)c0;
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                        : "r"(taddr));
                    if (KS > 1) {
                        // a split's partial sums, exact int32: [split][token][row]
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (row_ok) {
                            int32_t *pp = a.part + ((size_t)ks * a.S + s0) * a.O + o;
#pragma unroll
                            for (int j = 0; j < 16; j++)
                                if (s0 + j < a.S) pp[(size_t)j * a.O] = (int)r[j];
                        }
                    } else if (s0 + 16 <= a.S && !a.acc) {
                        // full chunk: the 16 token scales arrive while the accumulator is read; per token one
                        // conversion, two multiplies, one store of 32 consecutive rows
                        float sx[16];
                        const float4 *sx4 = reinterpret_cast<const float4 *>(a.sx + s0);
#pragma unroll
                        for (int j = 0; j < 4; j++) { float4 v = __ldg(sx4 + j); sx[4 * j] = v.x; sx[4 * j + 1] = v.y; sx[4 * j + 2] = v.z; sx[4 * j + 3] = v.w; }
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (row_ok) {
                            float *yp = a.y + (size_t)s0 * a.O + o;
#pragma unroll
                            for (int j = 0; j < 16; j++) yp[(size_t)j * a.O] = __fmul_rn(__fmul_rn(sc, sx[j]), (float)(int)r[j]);
                        }
                    } else {
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            int s = s0 + j;
                            if (s < a.S && row_ok) {
                                int v = (int)r[j];
                                a.y[(size_t)s * a.O + o] = __fmul_rn(__fmul_rn(sc, __ldg(a.sx + s)), (float)v);
                                if (a.acc) a.acc[(size_t)s * a.O + o] = v;
                            }
                        }
                    }
                }
            }
            // this warp is done reading the accumulator: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty_bar[buf])) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (abort_s) {
        // give bulk copies that may still be in flight time to land before the CTA's memory is released
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && abort_s) atomicExch(a.err, 1);
}

// y[s][o] = (scale[o] * sx[s]) * (float)(sum of the splits' int32 partials): the reference epilogue (nn/matmul.c:34)
__global__ void __launch_bounds__(256) tc_splitk_finish_kernel(const int32_t *__restrict__ part, int KS, const float *__restrict__ scale,
                                                               const float *__restrict__ sx, float *__restrict__ y,
                                                               int32_t *__restrict__ acc, int S, int O) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)S * O, i = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    int v = 0;
    for (int k = 0; k < KS; k++) v += part[(size_t)k * n + i];
    const int s = (int)(i / O), o = (int)(i - (size_t)s * O);
    y[i] = __fmul_rn(__fmul_rn(scale[o], sx[s]), (float)v);
    if (acc) acc[i] = v;
}

template <int BN, int STAGES, int MT>
int launch_tc_t(const CUtensorMap &mapA, const MotyCudaMat *w, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                int S, DevCtx *c, cudaStream_t st) {
    CUtensorMap mapB;
    CKR(make_map(&mapB, xi, S, w->I, BN));
    size_t smem = (size_t)STAGES * (MT * BM * BKB + BN * BKB) + 1024;
    auto k = q8_tc_kernel<BN, STAGES, MT>;
    CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    TcArgs a;
    a.scale = (const float *)w->scales; a.sx = sx; a.y = y; a.acc = acc; a.S = S; a.I = w->I; a.O = w->O; a.err = c->err_dev;
    int ntiles = ((w->O + MT * BM - 1) / (MT * BM)) * ((S + BN - 1) / BN);
    // few tiles and a long K: split K so that every SM streams a share of the weights
    const int nkb = (w->I + BKB - 1) / BKB;
    int ks = 1;
    // (measured on 3840 x 15360: 30 tiles 60 -> 31 us at S = 32..64; 60 tiles at S = 512 lose to the extra pass)
    if (ntiles * 4 <= c->sms && nkb >= 16) {
        ks = c->sms / ntiles;
        if (ks > 8) ks = 8;
        if (ks > nkb / 8) ks = nkb / 8;                         // at least 8 K blocks per split
        const int nks = (nkb + ks - 1) / ks;
        ks = (nkb + nks - 1) / nks;                             // no empty split
    }
    a.ksplit = ks; a.part = nullptr;
    if (ks > 1) {
        CKR(moty_grow(c, &c->pair, (size_t)ks * S * w->O * 4));
        a.part = (int32_t *)c->pair.p;
    }
    int work = ntiles * ks;
    int grid = work < c->sms ? work : c->sms;                  // persistent: one CTA per SM
    CK(moty_launch_pdl(k, dim3(grid), dim3(TC_THREADS), smem, st, mapA, mapB, a));
    if (ks > 1) {
        const size_t n = (size_t)S * w->O;
        CK(moty_launch_pdl(tc_splitk_finish_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, st,
                           (const int32_t *)a.part, ks, a.scale, sx, y, acc, S, w->O));
    }
    return 0;
}

}  // namespace

// the tensor map wants 16-byte row strides; rows shorter than one K block gain nothing
bool q8_tc_supported(int S, int I, int O) { return S >= 9 && I % 16 == 0 && I >= 128 && O >= 1; }

int q8_tc_make_tmap(MotyCudaMat *m) {
    m->has_tmap = false;
    if (m->fmt != MOTY_WF_I8 || m->I % 16 != 0 || m->I < 128) return 0;
    static_assert(sizeof(CUtensorMap) <= sizeof(m->tmap), "tensor map storage");
    if (make_map(reinterpret_cast<CUtensorMap *>(m->tmap), m->codes, m->O, m->I, BM) != 0) return 0;
    m->has_tmap = true;
    return 0;
}

int launch_q8_tc(const MotyCudaMat *w, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                 int S, DevCtx *c, cudaStream_t st) {
    const CUtensorMap &mapA = *reinterpret_cast<const CUtensorMap *>(w->tmap);
    if (S <= 16) return launch_tc_t<16, 8, 1>(mapA, w, xi, sx, y, acc, S, c, st);
    if (S <= 32) return launch_tc_t<32, 8, 1>(mapA, w, xi, sx, y, acc, S, c, st);
    if (S <= 64) return launch_tc_t<64, 6, 1>(mapA, w, xi, sx, y, acc, S, c, st);
    if (S <= 128) return launch_tc_t<128, 6, 1>(mapA, w, xi, sx, y, acc, S, c, st);
    // Large batches are bound by the bytes that reach shared memory per MAC, so the widest token
    // tile wins (measured on 15360x3840, S=4096: 256-token tiles 1.8-1.96 POP/s, 128-token tiles
    // 1.3); with few 128 x 256 tiles the batch is cut into 128-token tiles so that more SMs take
    // part.  The 256-row variant (MT = 2) halves the activation bytes per MAC but has no second
    // accumulator to overlap its epilogue and measured slower everywhere (1.3 POP/s): not selected.
    const long long t256 = (long long)((w->O + 127) / 128) * ((S + 255) / 256);
    if (t256 * 10 < (long long)c->sms * 6) return launch_tc_t<128, 6, 1>(mapA, w, xi, sx, y, acc, S, c, st);
    return launch_tc_t<256, 4, 1>(mapA, w, xi, sx, y, acc, S, c, st);
}
