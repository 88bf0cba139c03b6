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
};

DevCtx *moty_ctx(int device);                       // nullptr when not initialised
int moty_grow(DevCtx *c, Buf *b, size_t bytes);     // device buffer, grow-only
int moty_grow_pinned(DevCtx *c, Buf *b, size_t bytes);
int moty_grow_zero(DevCtx *c, Buf *b, size_t bytes);   // device buffer, zero-filled when (re)allocated

struct MotyCudaMat {
    int fmt, O, I, device;
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

#endif  // __CUDACC__
