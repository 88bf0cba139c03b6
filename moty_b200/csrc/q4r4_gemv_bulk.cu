// q4r4_gemv_bulk.cu -- the Q4R4 decode GEMV for matrices with few, long rows (FFN
// projections): one lane per weight row, fed by bulk asynchronous copies.
//
// A lane that owns a row runs the reference's chain without any shuffle
// (moty_hw_q4r4_gemm_ref, hw/hw_q4r4.h:47-63: exact integer sum per group of 32, then
// acc = fma((float)(sum - 8 * xsum), d * xs, acc) in ascending group order) in ~30
// instructions per group -- but a 3840 x 15360 matrix has only 120 warps of 32 rows, and 120
// warps cannot keep HBM busy from registers: each would need tens of KB in flight.  Here a warp
// is a CTA of its own and its eight 4-row blocks, which are eight contiguous streams in memory,
// arrive through cp.async.bulk into a ring of shared-memory stages (16 groups per stage, up to
// eight stages = 68 KB in flight per warp), tracked by one mbarrier per stage.  The same warp
// consumes a stage and re-arms it, so no second barrier is needed; every wait is bounded.
// The activation row is group-quantized once by quant_g32_kernel (quant.cu) and reaches every
// CTA with three more bulk copies.  Same bits as the other Q4R4 decode kernels.
#include "kernels.cuh"

namespace {

struct Q4GBArgs {
    const uint8_t *w; const uint16_t *d;
    const int8_t *xq; const float *xs; const int32_t *xsum;   // the group-quantized activation row
    float *y;
    int *err;
    int I, O, nst;                                            // nst: stages in the ring
};

constexpr int GB_G = 16;                          // groups per stage
constexpr int GB_WBLK = GB_G * 64 + 64;           // a block's codes in a stage, padded: two blocks of a quarter-warp read different banks
constexpr int GB_STAGE = 8 * GB_WBLK + 8 * GB_G * 8;
constexpr unsigned GB_WAIT_LIMIT = 1u << 26;

__device__ __forceinline__ unsigned gb_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gb_bulk(void *dst, const void *src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(gb_smem(dst)), "l"(src), "r"(bytes), "r"(gb_smem(bar)) : "memory");
}
__device__ __forceinline__ void gb_expect(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gb_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool gb_wait(unsigned long long *bar, unsigned parity) {
    return moty_mbar_wait_bounded(gb_smem(bar), parity, GB_WAIT_LIMIT);
}
__device__ __forceinline__ int dp4a_us3(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// one warp per CTA; unit = 32 consecutive rows = 8 blocks
__global__ void __launch_bounds__(32) q4r4_gemv_bulk_kernel(Q4GBArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int I = a.I, nb = I / 32, O = a.O, nst = a.nst;
    const int lane = threadIdx.x;
    const int nblk = (O + 3) / 4, blk0 = blockIdx.x * 8;
    int nblk_here = nblk - blk0; nblk_here = nblk_here < 8 ? nblk_here : 8;      // blocks of this unit that exist
    unsigned char *ring = smem;
    int8_t *xq_s = reinterpret_cast<int8_t *>(smem + (size_t)nst * GB_STAGE);
    float *xs_s = reinterpret_cast<float *>(xq_s + I);
    int *xsum_s = reinterpret_cast<int *>(xs_s + nb);
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(xsum_s + nb);   // nst stage barriers + 1 for the activation row
    const int nch = (nb + GB_G - 1) / GB_G;

    if (lane == 0) {
        for (int i = 0; i <= nst; i++)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(gb_smem(&bars[i])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // stage c % nst <- groups [c*16, c*16 + ng) of the unit's blocks: codes and f16 scales, one copy each per block
    auto fill = [&](int c) {
        const int g0 = c * GB_G, ng = nb - g0 < GB_G ? nb - g0 : GB_G;
        unsigned char *st = ring + (size_t)(c % nst) * GB_STAGE;
        unsigned long long *bar = &bars[c % nst];
        gb_expect(bar, (unsigned)(nblk_here * ng * (64 + 8)));
        for (int b = 0; b < nblk_here; b++) {
            const size_t cell = (size_t)(blk0 + b) * nb + g0;
            gb_bulk(st + b * GB_WBLK, a.w + cell * 64, (unsigned)(ng * 64), bar);
            gb_bulk(st + 8 * GB_WBLK + b * GB_G * 8, a.d + cell * 4, (unsigned)(ng * 8), bar);
        }
    };
    pdl_trigger();
    if (lane == 0) {
        for (int c = 0; c < nst && c < nch; c++) fill(c);                 // weights only: may overlap the previous kernel
    }
    pdl_wait();                                                           // the quantized row comes from the launch before this one
    if (lane == 0) {
        gb_expect(&bars[nst], (unsigned)(I + nb * 8));
        gb_bulk(xq_s, a.xq, (unsigned)I, &bars[nst]);
        gb_bulk(xs_s, a.xs, (unsigned)(nb * 4), &bars[nst]);
        gb_bulk(xsum_s, a.xsum, (unsigned)(nb * 4), &bars[nst]);
    }
    bool ok = gb_wait(&bars[nst], 0);

    const int bl = lane >> 2, r = lane & 3;
    float acc = 0.f;
    for (int c = 0; c < nch && ok; c++) {
        ok = gb_wait(&bars[c % nst], (unsigned)((c / nst) & 1));
        if (!ok) break;
        const unsigned char *st = ring + (size_t)(c % nst) * GB_STAGE;
        const unsigned char *wp = st + bl * GB_WBLK + r * 16;
        const unsigned char *dp = st + 8 * GB_WBLK + bl * GB_G * 8 + r * 2;
        const int g0 = c * GB_G, ng = nb - g0 < GB_G ? nb - g0 : GB_G;
        auto step = [&](int u) {
            const int g = g0 + u;
            const int4 w4 = *reinterpret_cast<const int4 *>(wp + u * 64);
            const int4 *xg = reinterpret_cast<const int4 *>(xq_s + (size_t)g * 32);
            const int4 x0 = xg[0], x1 = xg[1];
            // low nibbles as they are; high nibbles stay in place (16 x their value), are read as UNSIGNED bytes by
            // dp4a and the exact factor 16 is shifted out of the sum afterwards
            int sraw = __dp4a(w4.x & 0x0f0f0f0f, x0.x, 0);
            sraw = __dp4a(w4.y & 0x0f0f0f0f, x0.y, sraw);
            sraw = __dp4a(w4.z & 0x0f0f0f0f, x0.z, sraw);
            sraw = __dp4a(w4.w & 0x0f0f0f0f, x0.w, sraw);
            int s16 = dp4a_us3((unsigned)w4.x & 0xf0f0f0f0u, x1.x, 0);
            s16 = dp4a_us3((unsigned)w4.y & 0xf0f0f0f0u, x1.y, s16);
            s16 = dp4a_us3((unsigned)w4.z & 0xf0f0f0f0u, x1.z, s16);
            s16 = dp4a_us3((unsigned)w4.w & 0xf0f0f0f0u, x1.w, s16);
            sraw += s16 >> 4;
            const float dd = f16bits_to_f32(*reinterpret_cast<const uint16_t *>(dp + u * 8));
            // token-by-token formula (hw/hw_q4r4.h:58-59)
            acc = fmaf((float)(sraw - 8 * xsum_s[g]), __fmul_rn(dd, xs_s[g]), acc);
        };
        if (ng == GB_G) {
#pragma unroll
            for (int u = 0; u < GB_G; u++) step(u);
        } else {
            for (int u = 0; u < ng; u++) step(u);
        }
        __syncwarp();                                                     // every lane is done with this stage
        if (lane == 0 && c + nst < nch) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic reads before the async overwrite
            fill(c + nst);
        }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
        // a bounded wait expired: copies may still be in flight towards this CTA's memory; give them time, report
        for (int i = 0; i < 1000; i++) __nanosleep(1000);
        if (lane == 0) atomicExch(a.err, 1);
        return;
    }
    const int row = blockIdx.x * 32 + lane;
    if (row < O) a.y[row] = acc;
}

}  // namespace

// few enough rows that a lane-per-row kernel from registers would starve (q4r4_gemv1.cu takes the others), enough
// of them for two or more warps per SM (with one warp per SM the kernel is bound by that warp's instruction
// issue: 3840 x 15360 measured 41.6 us against 37.7 us of q4r4_stream_kernel, 15360 x 3840 19.5 against 23.0),
// rows long enough for a ring, copy sizes multiples of 16 bytes
bool q4r4_gemv_bulk_supported(int I, int O, int sms) {
    const int nunits = ((O + 3) / 4 + 7) / 8;
    return I % 128 == 0 && I >= 1024 && I <= MOTY_QROW_MAX && nunits >= sms * 2 && nunits < sms * 12 &&
           (long long)((O + 3) / 4) * (I / 32) >= 400000;          // big enough to be worth a second launch (the quantizer)
}

size_t q4r4_gemv_bulk_smem(int I, int nst) {
    return (size_t)nst * GB_STAGE + (size_t)I + (size_t)(I / 32) * 8 + (size_t)(nst + 1) * 8 + 128;
}

// xq/xs/xsum: the activation row group-quantized by launch_quant_g32 (same stream, just before)
int launch_q4r4_gemv_bulk(const uint8_t *w, const uint16_t *d, const int8_t *xq, const float *xs, const int32_t *xsum,
                          float *y, int I, int O, int *err, int sms, cudaStream_t st) {
    if (!q4r4_gemv_bulk_supported(I, O, sms)) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv_bulk: I=%d O=%d", I, O);
    const int nunits = ((O + 3) / 4 + 7) / 8, nch = (I / 32 + GB_G - 1) / GB_G;
    // ring depth: as many stages as fit when every SM holds its share of the units (at most 8, at most the row)
    const int per_sm = (nunits + sms - 1) / sms;
    int nst = 8;
    while (nst > 2 && (q4r4_gemv_bulk_smem(I, nst) + 1024) * per_sm > 200 * 1024) nst--;
    if (nst > nch) nst = nch;
    const size_t smem = q4r4_gemv_bulk_smem(I, nst);
    if (smem > 200 * 1024) return moty_set_error(MOTY_CUDA_ELIMIT, "q4r4_gemv_bulk: I=%d needs %zu bytes of shared memory", I, smem);
    static size_t attr_smem[MOTY_MAX_DEV];
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q4r4_gemv_bulk: device %d", dev);
    if (smem > attr_smem[dev]) {
        CK(cudaFuncSetAttribute(q4r4_gemv_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev] = smem;
    }
    Q4GBArgs a; a.w = w; a.d = d; a.xq = xq; a.xs = xs; a.xsum = xsum; a.y = y; a.err = err; a.I = I; a.O = O; a.nst = nst;
    CK(moty_launch_pdl(q4r4_gemv_bulk_kernel, dim3(nunits), dim3(32), smem, st, a));
    return 0;
}
