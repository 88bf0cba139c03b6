// noalloc.cu -- a Q8_0 product that never allocates.
//
// Some hosts cannot let a library call cudaMalloc once they are running: a
// serving process that has handed the whole HBM budget to its own pool, or a
// decode loop that cannot afford the device-wide synchronisation cudaMalloc and
// cudaFree imply.  For them this file offers one entry that keeps its scratch
// (the int8 codes and the scales of the activation rows between the quantizer
// kernel and the product kernel) in a fixed array linked into the library.
// Every GPU that loads the library carries that array (about 128 KB) until the
// process exits.
//
// The array's name is only a host-side handle: passing it to a kernel would hand
// the kernel a host address.  Host code therefore asks the runtime for the
// device address once per device (cudaGetSymbolAddress, with that device
// current) and passes that pointer on.
#include "kernels.cuh"

#define NOALLOC_MAX_S 8
#define NOALLOC_MAX_I MOTY_QROW_MAX

// [8][16384] int8 codes, then 8 f32 scales (256-byte aligned sub-blocks)
static __device__ __align__(256) unsigned char g_q8_noalloc_scratch[NOALLOC_MAX_S * NOALLOC_MAX_I + 256];

static void *g_scratch_ptr[MOTY_MAX_DEV];
static int g_sms[MOTY_MAX_DEV];
static bool g_ready[MOTY_MAX_DEV];

// once per device: device address of the scratch, SM count, kernel attributes; allocates nothing
static int noalloc_setup(int device) {
    if (g_ready[device]) return 0;
    void *p = nullptr;
    CK(cudaGetSymbolAddress(&p, g_q8_noalloc_scratch));
    if (!p) return moty_set_error(MOTY_CUDA_ECUDA, "noalloc: scratch symbol has no device address");
    int sms = 0, major = 0;
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    CK(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return moty_set_error(MOTY_CUDA_EINIT, "noalloc: device %d is not sm_100", device);
    CKR(gemv_q8_init_device());
    g_scratch_ptr[device] = p; g_sms[device] = sms; g_ready[device] = true;
    return 0;
}

extern "C" int moty_cuda_q8_apply_noalloc(float *y_dev, const float *x_dev, const int8_t *q_dev, const float *scale_dev,
                                          int S, int I, int O, int device, void *stream) {
    if (!y_dev || !x_dev || !q_dev || !scale_dev) return moty_set_error(MOTY_CUDA_EARG, "q8_apply_noalloc: null pointer");
    if (S < 1 || S > NOALLOC_MAX_S)
        return moty_set_error(MOTY_CUDA_ELIMIT, "q8_apply_noalloc: S=%d, this entry takes 1..%d rows (its scratch is fixed)", S, NOALLOC_MAX_S);
    if (I < 16 || I > NOALLOC_MAX_I || I % 16)
        return moty_set_error(MOTY_CUDA_ELIMIT, "q8_apply_noalloc: I=%d, this entry takes multiples of 16 up to %d", I, NOALLOC_MAX_I);
    if (O < 1) return moty_set_error(MOTY_CUDA_EARG, "q8_apply_noalloc: O=%d", O);
    // the product kernel reads the weights with 16-byte loads; unlike the matrices the library uploads itself, these
    // pointers are the caller's and may be slices: refuse before any launch instead of faulting on the GPU
    if (reinterpret_cast<uintptr_t>(q_dev) & 15)
        return moty_set_error(MOTY_CUDA_EARG, "q8_apply_noalloc: q_dev must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(y_dev) | reinterpret_cast<uintptr_t>(x_dev) | reinterpret_cast<uintptr_t>(scale_dev)) & 3)
        return moty_set_error(MOTY_CUDA_EARG, "q8_apply_noalloc: y_dev, x_dev and scale_dev must be 4-byte aligned");
    if (device < 0 || device >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "q8_apply_noalloc: device %d", device);
    MOTY_USE_DEVICE(device);                       // the caller's current device is put back on return
    CKR(noalloc_setup(device));
    cudaStream_t st = (cudaStream_t)stream;
    int8_t *xi = (int8_t *)g_scratch_ptr[device];
    float *sx = (float *)((char *)g_scratch_ptr[device] + (size_t)NOALLOC_MAX_S * NOALLOC_MAX_I);
    // nothing in the scratch has to start at zero: the quantizer rewrites every byte the product reads
    CKR(launch_qrow_i8(x_dev, xi, sx, S, I, st));
    Q8Args a;
    a.w = q_dev; a.scale = scale_dev; a.tiles = nullptr; a.ntiles_dev = nullptr; a.ntiles_max = 0;
    a.xi = xi; a.sx = sx; a.xmap = nullptr; a.ymap = nullptr;
    a.y = y_dev; a.ldy = O; a.acc = nullptr; a.S = S; a.I = I; a.O = O;
    return launch_q8_small(a, g_sms[device], st);
}
