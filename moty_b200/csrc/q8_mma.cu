// q8_mma.cu -- Q8_0 weights x a small batch of quantized activation rows (9 <= S <= 64), and
// the grouped products of a MoE batch with int8 experts.
//
// Replaces moty_matmul_q_s (nn/matmul.c:51-66, IDOT=1) for batches too small to fill a
// 128 x N tcgen05 tile economically: there the product is bound by streaming the weights once,
// and the 5th-generation tensor-core kernel (gemm_q8_tc.cu) spends its time on tile
// fill and drain.  Here a CTA streams 128 weight rows through a four-stage cp.async ring
// (128 bytes of K per row and stage, rows padded to 144 bytes so that the eight rows of a fragment
// load sit in different banks) and every warp feeds its 16 rows to mma.sync.m16n8k32
// (s8 x s8 -> s32); the int32 accumulators stay in registers over the whole row, so the result
// is the exact integer dot of the reference and the epilogue is its
// (scale[o] * sx[s]) * (float)acc, left to right (nn/matmul.c:34).
#include "kernels.cuh"
#include <string.h>

struct Q8MmaArgs {
    const int8_t *w; const float *scale;       // dense: [O][I], [O]
    const int8_t *xi; const float *sx;         // activation codes [..][I] and row scales
    float *y; int32_t *acc; int ldy;
    int S, I, O;
    // grouped mode: CTA row y of the grid is a tile = up to 8 NT consecutive rows of the gathered
    // batch that share one expert's matrix; activation rows are found through xmap (null: identity)
    const Q8Tile *tiles; const int *ntiles_dev; const int *xmap;
    // dense split-K: grid.z CTAs share a tile's K range; their int32 partials meet in part[S][O] (zero between calls),
    // the CTA that arrives last at ctr[tile] (zero between calls) writes the result and leaves both zero again
    int ksplit; int32_t *part; unsigned *ctr;
};

__device__ __forceinline__ void mma_s8s8_16832(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int Q8M_KCH = 128, Q8M_ROW = Q8M_KCH + 16, Q8M_NSTG = 4;
template <int NT> struct Q8MStage {
    static constexpr int W = 0, B = 128 * Q8M_ROW, BYTES = B + NT * 8 * Q8M_ROW;
};

template <int NT>
__global__ void __launch_bounds__(256) q8_mma_kernel(Q8MmaArgs a) {
    using L = Q8MStage<NT>;
    extern __shared__ int4 smem_q8mma[];
    unsigned char *smem = reinterpret_cast<unsigned char *>(smem_q8mma);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, tid = lane & 3;
    const int I = a.I, O = a.O;
    const int8_t *Wp = a.w; const float *Sc = a.scale;
    int n00 = blockIdx.y * NT * 8, S = a.S;
    pdl_trigger();
    if (a.tiles) {
        pdl_wait();                                            // the tile table comes from the plan kernel
        if ((int)blockIdx.y >= *a.ntiles_dev) return;          // CTA-uniform
        const Q8Tile t = a.tiles[blockIdx.y];
        Wp = t.w; Sc = t.scale; n00 = t.row0; S = t.row0 + t.nrows;
    }
    const int row0 = blockIdx.x * 128;
    const int nstage_all = (I + Q8M_KCH - 1) / Q8M_KCH;
    // this CTA's share of the K stages (dense split-K; otherwise everything)
    const int per_z = (nstage_all + (int)gridDim.z - 1) / (int)gridDim.z;
    const int s_lo = (int)blockIdx.z * per_z, nstage = nstage_all - s_lo < per_z ? (nstage_all - s_lo > 0 ? nstage_all - s_lo : 0) : per_z;
    // copies: a row's 128 bytes of a stage are 8 chunks of 16; thread t takes chunk t & 7 of rows t >> 3, + 32, ...
    const int ch = threadIdx.x & 7, r_first = threadIdx.x >> 3;
    auto fill_w = [&](int s) {
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % Q8M_NSTG) * L::BYTES + L::W;
        const int k = (s_lo + s) * Q8M_KCH + ch * 16;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const int r = r_first + q * 32;
            int row = row0 + r; row = row < O ? row : O - 1;   // rows past the end: a valid row, nothing stored
            cp_async16_zfill(dst + r * Q8M_ROW + ch * 16, Wp + (size_t)row * I + (k < I ? k : 0), k < I);
        }
    };
    auto fill_x = [&](int s) {
        if (s >= nstage) return;
        unsigned char *dst = smem + (size_t)(s % Q8M_NSTG) * L::BYTES + L::B;
        const int k = (s_lo + s) * Q8M_KCH + ch * 16;
        for (int r = r_first; r < NT * 8; r += 32) {
            int n = n00 + r; n = n < S ? n : S - 1;
            if (a.xmap) n = a.xmap[n];
            cp_async16_zfill(dst + r * Q8M_ROW + ch * 16, a.xi + (size_t)n * I + (k < I ? k : 0), k < I);
        }
    };
    fill_w(0); fill_w(1); fill_w(2);                           // weights only: may overlap the previous kernel
    pdl_wait();                                                // activation codes come from the quantizer launch
    fill_x(0); cp_async_commit();
    fill_x(1); cp_async_commit();
    fill_x(2); cp_async_commit();

    int acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0;
    const int offA = (warp * 16 + gid) * Q8M_ROW + tid * 4, offB = gid * Q8M_ROW + tid * 4;
    for (int s = 0; s < nstage; s++) {
        cp_async_wait<2>();                                    // this thread's copies of stage s have landed
        __syncthreads();                                       // everyone's have, and everyone is done with stage s - 1
        fill_w(s + 3); fill_x(s + 3); cp_async_commit();       // into the slot stage s - 1 used
        const unsigned char *st = smem + (size_t)(s % Q8M_NSTG) * L::BYTES;
#pragma unroll
        for (int kk = 0; kk < Q8M_KCH / 32; kk++) {
            const unsigned char *ap = st + L::W + offA + kk * 32;
            const unsigned a0 = *reinterpret_cast<const unsigned *>(ap), a2 = *reinterpret_cast<const unsigned *>(ap + 16);
            const unsigned a1 = *reinterpret_cast<const unsigned *>(ap + 8 * Q8M_ROW), a3 = *reinterpret_cast<const unsigned *>(ap + 8 * Q8M_ROW + 16);
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const unsigned char *bp = st + L::B + j * 8 * Q8M_ROW + offB + kk * 32;
                mma_s8s8_16832(acc[j], a0, a1, a2, a3, *reinterpret_cast<const unsigned *>(bp), *reinterpret_cast<const unsigned *>(bp + 16));
            }
        }
    }
    cp_async_wait<0>();
    const int ra = row0 + warp * 16 + gid, rb = ra + 8;
    if (gridDim.z > 1) {
        // integer partials are exact in any order: add them up in global memory, the last CTA of the tile finishes
        __shared__ unsigned s_last;
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int t = n00 + j * 8 + tid * 2 + h;
                if (t >= S) continue;
                if (ra < O) atomicAdd(a.part + (size_t)t * O + ra, acc[j][h]);
                if (rb < O) atomicAdd(a.part + (size_t)t * O + rb, acc[j][2 + h]);
            }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const unsigned tile = blockIdx.y * gridDim.x + blockIdx.x;
            const unsigned prev = atomicAdd(a.ctr + tile, 1u);
            s_last = prev == gridDim.z - 1;
            if (s_last) a.ctr[tile] = 0;                       // ready for the next call
        }
        __syncthreads();
        if (!s_last) return;
        __threadfence();
#pragma unroll
        for (int j = 0; j < NT; j++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int t = n00 + j * 8 + tid * 2 + h;
                if (t >= S) continue;
                if (ra < O) { acc[j][h] = __ldcg(a.part + (size_t)t * O + ra); a.part[(size_t)t * O + ra] = 0; }
                if (rb < O) { acc[j][2 + h] = __ldcg(a.part + (size_t)t * O + rb); a.part[(size_t)t * O + rb] = 0; }
            }
        }
    }
    const float sa = ra < O ? Sc[ra] : 0.f, sb = rb < O ? Sc[rb] : 0.f;
#pragma unroll
    for (int j = 0; j < NT; j++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int t = n00 + j * 8 + tid * 2 + h;
            if (t >= S) continue;
            const float sx = a.sx[a.xmap ? a.xmap[t] : t];
            if (ra < O) {
                a.y[(size_t)t * a.ldy + ra] = __fmul_rn(__fmul_rn(sa, sx), (float)acc[j][h]);
                if (a.acc) a.acc[(size_t)t * a.ldy + ra] = acc[j][h];
            }
            if (rb < O) {
                a.y[(size_t)t * a.ldy + rb] = __fmul_rn(__fmul_rn(sb, sx), (float)acc[j][2 + h]);
                if (a.acc) a.acc[(size_t)t * a.ldy + rb] = acc[j][2 + h];
            }
        }
    }
}

template <int NT>
static int launch_q8m_t(const Q8MmaArgs &a, cudaStream_t st, int ntiles_max) {
    constexpr int SMEM = Q8M_NSTG * Q8MStage<NT>::BYTES;
    static bool attr_done[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q8_mma: device %d", dev);
    if (!attr_done[dev]) {
        CK(cudaFuncSetAttribute(q8_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        attr_done[dev] = true;
    }
    dim3 grid((a.O + 127) / 128, a.tiles ? ntiles_max : (a.S + 8 * NT - 1) / (8 * NT), a.tiles || a.ksplit < 2 ? 1 : a.ksplit);
    if (grid.y > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "q8_mma: %u token tiles in one call", grid.y);
    CK(moty_launch_pdl(q8_mma_kernel<NT>, grid, dim3(256), (size_t)SMEM, st, a));
    return 0;
}

bool q8_mma_supported(int S, int I, int O) { return S >= 1 && I % 16 == 0 && I >= 16 && O >= 1; }

// K splits worth taking for a dense product: none while the row and token tiles alone give every SM a CTA (the
// partials cost one atomic per output and split: 15360 x 3840 at S = 16, 240 CTAs, lost 6 us to a split in two);
// else enough for two CTAs per SM, at most 8, each with at least 8 stages (5120 x 13824 at S = 12: 45.7 -> 35.7 us,
// 1024 x 3072 at S = 16: 16.4 -> 10.5 us)
int q8_mma_ksplit(int S, int I, int O, int sms) {
    const long long mct = (O + 127) / 128, want = (long long)sms * 2;
    const int nt = S > 16 && mct * ((S + 31) / 32) >= want ? 4 : (S > 8 && mct * ((S + 15) / 16) >= want ? 2 : 1);
    const long long ctas = mct * ((S + 8 * nt - 1) / (8 * nt));
    const int nstage = (I + Q8M_KCH - 1) / Q8M_KCH;
    if (ctas >= sms || nstage < 16) return 1;
    int ks = (int)((want + ctas - 1) / ctas);
    if (ks > 8) ks = 8;
    if (ks > nstage / 8) ks = nstage / 8;
    return ks < 2 ? 1 : ks;
}

// scratch for split-K: S * O int32 partials after 4096 tile counters, all zero between calls
size_t q8_mma_scratch_bytes(int S, int O) { return 4096 * 4 + (size_t)S * O * 4; }

// xi/sx: the S quantized rows.  y (and acc, optional) [S][O].  scratch: null, or q8_mma_scratch_bytes(S, O) zero-filled
// bytes that stay zero from call to call (allows split-K, see q8_mma_ksplit).
int launch_q8_mma(const int8_t *w, const float *scale, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                  int S, int I, int O, void *scratch, int sms, cudaStream_t st) {
    if (!q8_mma_supported(S, I, O)) return moty_set_error(MOTY_CUDA_EARG, "q8_mma: S=%d I=%d O=%d", S, I, O);
    Q8MmaArgs a; memset(&a, 0, sizeof a);
    a.w = w; a.scale = scale; a.xi = xi; a.sx = sx; a.y = y; a.acc = acc; a.ldy = O; a.S = S; a.I = I; a.O = O;
    // wider token tiles read the weights fewer times; narrower ones give more CTAs
    const long long mct = (O + 127) / 128, want = (long long)sms * 2;
    const int nt = S > 16 && mct * ((S + 31) / 32) >= want ? 4 : (S > 8 && mct * ((S + 15) / 16) >= want ? 2 : 1);
    a.ksplit = 1;
    if (scratch && mct * ((S + 8 * nt - 1) / (8 * nt)) <= 4096) {
        a.ksplit = q8_mma_ksplit(S, I, O, sms);
        a.ctr = reinterpret_cast<unsigned *>(scratch);
        a.part = reinterpret_cast<int32_t *>(reinterpret_cast<unsigned char *>(scratch) + 4096 * 4);
    }
    if (nt == 4) return launch_q8m_t<4>(a, st, 0);
    if (nt == 2) return launch_q8m_t<2>(a, st, 0);
    return launch_q8m_t<1>(a, st, 0);
}

// Grouped products of a MoE batch: tiles[i] = {expert matrix, first row, rows <= tile_rows} over a
// gathered batch; activation row p is row xmap[p] (null: p) of xi/sx; y row p receives the product.
int launch_q8_mma_grouped(const Q8Tile *tiles, const int *ntiles_dev, int ntiles_max, int tile_rows,
                          const int8_t *xi, const float *sx, const int *xmap, float *y, int ldy, int I, int O,
                          cudaStream_t st) {
    if (I % 16 != 0 || I < 16 || (tile_rows != 8 && tile_rows != 16 && tile_rows != 32))
        return moty_set_error(MOTY_CUDA_EARG, "q8_mma_grouped: I=%d tile=%d", I, tile_rows);
    if (O <= 0 || ntiles_max <= 0) return 0;
    if (ntiles_max > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "q8_mma_grouped: %d tiles in one call", ntiles_max);
    Q8MmaArgs a; memset(&a, 0, sizeof a);
    a.xi = xi; a.sx = sx; a.y = y; a.ldy = ldy; a.I = I; a.O = O;
    a.tiles = tiles; a.ntiles_dev = ntiles_dev; a.xmap = xmap;
    if (tile_rows == 32) return launch_q8m_t<4>(a, st, ntiles_max);
    if (tile_rows == 16) return launch_q8m_t<2>(a, st, ntiles_max);
    return launch_q8m_t<1>(a, st, ntiles_max);
}
