// common.cuh -- shared state and device helpers of libmoty_cuda (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/moty_cuda.h"

#define MOTY_MAX_DEV 16
#define MOTY_QROW_MAX 16384          // NN_QROW_MAX, nn/nn_matmul.h:35

// ---------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------
int moty_set_error(int code, const char *fmt, ...);

#define CK(call)                                                                       \
    do {                                                                               \
        cudaError_t e_ = (call);                                                       \
        if (e_ != cudaSuccess)                                                         \
            return moty_set_error(e_ == cudaErrorMemoryAllocation ? MOTY_CUDA_ENOMEM   \
                                                                  : MOTY_CUDA_ECUDA,   \
                                  "%s:%d %s: %s", __FILE__, __LINE__, #call,           \
                                  cudaGetErrorString(e_));                             \
    } while (0)

// With MOTY_CUDA_DEBUG_SYNC=1 in the environment every step of a driver is followed by a device
// synchronisation, so that a kernel fault is reported at the step that caused it (a debugging aid;
// it serialises everything and is off by default).
bool moty_debug_sync();

#define CKR(call)                                                                      \
    do {                                                                               \
        int r_ = (call);                                                               \
        if (r_ != 0) return r_;                                                        \
        if (moty_debug_sync()) {                                                       \
            cudaError_t e_ = cudaDeviceSynchronize();                                  \
            if (e_ != cudaSuccess)                                                     \
                return moty_set_error(MOTY_CUDA_ECUDA, "%s:%d after %s: %s", __FILE__, __LINE__, #call, \
                                      cudaGetErrorString(e_));                         \
        }                                                                              \
    } while (0)

// ---------------------------------------------------------------------------
// per-device context: one stream, grow-only scratch, pinned staging
// ---------------------------------------------------------------------------
struct Buf {
    void *p = nullptr;
    size_t cap = 0;
};

struct DevCtx {
    int dev = -1;
    bool ready = false;
    int sms = 0;
    cudaStream_t stream = nullptr;
    // activation scratch of the drivers (the reference's function-level statics)
    Buf xi, sx, xs, xsum, acc32;
    // staging for the host-pointer entries
    Buf dx, dy, dlogits, daux;
    Buf hpin_in, hpin_out;           // pinned host
    // FFN / MoE intermediates
    Buf g, u, h, hq, hs, hxs, hxsum, pair, misc;
    Buf rec;                         // per (token, group) records of the Q4R4 batch kernel
    Buf attn;                        // partial results of an attention call whose positions are split over CTAs
    Buf ffn1;                        // the constant logit and the index/weight outputs of a dense FFN run as a one-expert MoE block
    Buf mmak;                        // split-K scratch of the Q8_0 MMA kernel: tile counters + int32 partials, zero between calls
    // streaming GEMV: ticket/exit counters and K-split cells, all zero between launches
    int *ctr = nullptr;
    Buf kcell;
    // device error word written by kernels whose bounded waits expire
    int *err_dev = nullptr;
    // set by moty_cuda_scratch_freeze: the grow-only buffers may no longer move (a captured CUDA graph holds their addresses)
    bool frozen = false;
    // host-pointer entries with pinned buffers (hostio.cu): a pinned flag word the last kernel of a call writes, its
    // device alias, and the sequence number of the latest call
    unsigned *hflag = nullptr, *hflag_dev = nullptr, hseq = 0;
    // bumped whenever a scratch buffer of this device moves: cached graphs of host calls hold scratch addresses
    unsigned long long gen = 0;
};

// Every entry point that makes a GPU current puts the caller's device back before it returns.
struct MotyDevGuard {
    int prev = -1;
    cudaError_t set(int device) {
        if (prev < 0) {
            cudaError_t e = cudaGetDevice(&prev);
            if (e != cudaSuccess) { prev = -1; return e; }
        }
        return cudaSetDevice(device);
    }
    ~MotyDevGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
#define MOTY_CAT2(a, b) a##b
#define MOTY_CAT(a, b) MOTY_CAT2(a, b)
// make `device` current for the rest of the enclosing scope
#define MOTY_USE_DEVICE(device) MotyDevGuard MOTY_CAT(moty_dg_, __LINE__); CK(MOTY_CAT(moty_dg_, __LINE__).set(device))

DevCtx *moty_ctx(int device);                       // nullptr when not initialised
int moty_grow(DevCtx *c, Buf *b, size_t bytes);     // device buffer, grow-only
int moty_grow_pinned(DevCtx *c, Buf *b, size_t bytes);
int moty_grow_zero(DevCtx *c, Buf *b, size_t bytes);   // device buffer, zero-filled when (re)allocated

struct MotyCudaMat {
    int fmt, O, I, device;
    int src_fmt;        // the format it was uploaded in when that differs from fmt (WF_I4 rows are kept as WF_I8 codes), else 0
    void *codes;        // device
    void *scales;       // device
    size_t code_bytes, scale_bytes;
    // TMA descriptor of the int8 codes (WF_I8, I % 128 == 0), built at upload
    alignas(64) unsigned char tmap[128];
    bool has_tmap;
};

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// Programmatic dependent launch.  A kernel launched through moty_launch_pdl may start while the
// kernel before it on the stream is still draining; everything it does before pdl_wait() must
// touch only memory that no kernel writes (uploaded weights, its own shared memory), and every
// read of an activation and every global write comes after pdl_wait(), which returns once the
// earlier kernels have finished and their writes are visible.  pdl_trigger() lets the kernel
// after this one be scheduled into SMs as this one's CTAs leave.  Both are no-ops in a launch
// without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

bool moty_pdl_enabled();             // false when the environment has MOTY_CUDA_PDL=0

template <typename... KArgs, typename... Args>
inline cudaError_t moty_launch_pdl(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                   Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = moty_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k, static_cast<KArgs>(args)...);
}

// 16-, 8- and 4-byte asynchronous copies global -> shared (.cg: around L1, for data read once);
// cp_async16_zfill copies nothing and writes 16 zero bytes when !valid (the source is not read)
__device__ __forceinline__ void cp_async16(void *smem, const void *g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async16_zfill(void *smem, const void *g, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g),
                 "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem, const void *g) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async8(void *smem, const void *g) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((unsigned)__cvta_generic_to_shared(smem)), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ int4 ldg_stream16(const void *p) {
    // weights are read exactly once: keep them out of L1
    int4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ int warp_sum_i32(int v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

__device__ __forceinline__ float warp_max_f32(float v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}

__device__ __forceinline__ int dp4a4(const int4 &a, const int4 &b, int acc) {
    acc = __dp4a(a.x, b.x, acc);
    acc = __dp4a(a.y, b.y, acc);
    acc = __dp4a(a.z, b.z, acc);
    acc = __dp4a(a.w, b.w, acc);
    return acc;
}

// The activation quantizer step of moty_hw_qrow_i8 / moty_hw_quant_g32
// (hw/hw_quant.h:12-14, hw/hw_q4r4.h:40-42) with correctly rounded IEEE ops so
// that the codes equal the CPU's: s = amax/127 floored, inv = 1/s,
// q = rint(x*inv) (round-half-even; the explicit _rn multiply cannot be fused).
__device__ __forceinline__ float quant_scale(float amax, float floor_) {
    float s = __fdiv_rn(amax, 127.f);
    return s < floor_ ? floor_ : s;
}
__device__ __forceinline__ int quant_code(float x, float inv) {
    return __float2int_rn(__fmul_rn(x, inv));
}

__device__ __forceinline__ float f16bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));     // exact, subnormals included
}

// expf as the reference's C library computes it.  The reference calls libm's expf in SiLU, in the
// router softmax and in the output gate (hw/hw_ops.h:19-26, nn/moe.c:11,120,197, nn/attn.c:69), and an
// ulp of difference there can move an int8 code of the re-quantized hidden row.  glibc's expf (2.27 and
// later; the table-driven double-precision algorithm of ARM's optimized routines) is
//   z = x * 32/ln2;  k = round(z);  r = z - k;  2^(k/32) from a 32-entry table and the exponent field;
//   exp(x) = 2^(k/32) * (C0 r^3 + C1 r^2 + C2 r + 1) in f64, rounded ONCE to f32,
// and x86-64 hosts with FMA run the build in which the compiler contracted the multiply-adds:
// r = fma(32/ln2, x, -k) and the three polynomial steps below.  The same sequence written in C for the
// CPU checker equals the host's expf on every one of the 2^32 float inputs (the test-suite checks a
// sample of them in each run); IEEE f64 operations give the same bits here.  Entry i of the table is bits(2^(i/32) rounded to f64) - (i << 47).

__device__ __forceinline__ float moty_expf(float x) {
    static constexpr unsigned long long MOTY_EXP2_TAB[32] = {
        0x3ff0000000000000ULL, 0x3fefd9b0d3158574ULL, 0x3fefb5586cf9890fULL, 0x3fef9301d0125b51ULL,
        0x3fef72b83c7d517bULL, 0x3fef54873168b9aaULL, 0x3fef387a6e756238ULL, 0x3fef1e9df51fdee1ULL,
        0x3fef06fe0a31b715ULL, 0x3feef1a7373aa9cbULL, 0x3feedea64c123422ULL, 0x3feece086061892dULL,
        0x3feebfdad5362a27ULL, 0x3feeb42b569d4f82ULL, 0x3feeab07dd485429ULL, 0x3feea47eb03a5585ULL,
        0x3feea09e667f3bcdULL, 0x3fee9f75e8ec5f74ULL, 0x3feea11473eb0187ULL, 0x3feea589994cce13ULL,
        0x3feeace5422aa0dbULL, 0x3feeb737b0cdc5e5ULL, 0x3feec49182a3f090ULL, 0x3feed503b23e255dULL,
        0x3feee89f995ad3adULL, 0x3feeff76f2fb5e47ULL, 0x3fef199bdd85529cULL, 0x3fef3720dcef9069ULL,
        0x3fef5818dcfba487ULL, 0x3fef7c97337b9b5fULL, 0x3fefa4afa2a490daULL, 0x3fefd0765b6e4540ULL};
    const unsigned top = (__float_as_uint(x) >> 20) & 0x7ffu;
    if (top >= 0x42bu) {                                              // |x| >= 88, infinities and NaN
        if (__float_as_uint(x) == 0xff800000u) return 0.f;
        if (top >= 0x7f8u) return __fadd_rn(x, x);
        if (x > 0x1.62e42ep6f) return __int_as_float(0x7f800000);
        if (x < -0x1.9fe368p6f) return 0.f;
    }
    constexpr double INV_LN2_N = 0x1.71547652b82fep+0 * 32.0;
    constexpr double C0 = 0x1.c6af84b912394p-5 / 32 / 32 / 32, C1 = 0x1.ebfce50fac4f3p-3 / 32 / 32, C2 = 0x1.62e42ff0c52d6p-1 / 32;
    constexpr double SHIFT = 0x1.8p52;
    const double xd = (double)x;
    const double z = __dmul_rn(INV_LN2_N, xd);
    double kd = __dadd_rn(z, SHIFT);
    const unsigned long long ki = (unsigned long long)__double_as_longlong(kd);
    kd = __dsub_rn(kd, SHIFT);
    const double r = __fma_rn(INV_LN2_N, xd, -kd);
    const double s = __longlong_as_double((long long)(MOTY_EXP2_TAB[ki & 31] + (ki << 47)));
    const double p = __fma_rn(C0, r, C1);
    const double r2 = __dmul_rn(r, r);
    double y = __fma_rn(C2, r, 1.0);
    y = __fma_rn(p, r2, y);
    return __double2float_rn(__dmul_rn(y, s));
}
// SiLU(v) * u as the reference spells it: (v / (1 + expf(-v))) * u, three correctly rounded f32 steps
__device__ __forceinline__ float moty_silu_mul(float v, float u) {
    return __fmul_rn(__fdiv_rn(v, __fadd_rn(1.f, moty_expf(-v))), u);
}
// tanh-GeLU(v) * u as engines/gemma.c:389-391,398 spells it: 0.5 v (1 + tanhf(0.79788456 (v + 0.044715 v^3))) * u.
// v + 0.044715 v v v: the CPU build fuses the last multiply with the add; tanh is evaluated in f64 and rounded once.
__device__ __forceinline__ float moty_gelu_mul(float v, float u) {
    const float inner = __fmul_rn(0.7978845608028654f, fmaf(__fmul_rn(__fmul_rn(0.044715f, v), v), v, v));
    const float th = (float)tanh((double)inner);
    return __fmul_rn(__fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.f, th)), u);
}

#endif  // __CUDACC__
