// api.cu -- the C ABI of libmoty_cuda (include/moty_cuda.h): contexts, weight
// upload, the mat_apply / FFN / MoE drivers.  Host logic only; kernels live in
// the other translation units.  No CPU fallback anywhere: a failure is returned.
#include "kernels.cuh"
#include "moe.cuh"
#include <string.h>
#include <stdlib.h>
#include <new>

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int moty_set_error(int code, const char *fmt, ...) {
    va_list ap; va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char *moty_cuda_last_error(void) { return g_err; }

bool moty_debug_sync() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("MOTY_CUDA_DEBUG_SYNC");
        on = (e && e[0] == '1') ? 1 : 0;
    }
    return on == 1;
}

static int g_q4r4_relaxed = 0;  // Q4R4 / Q8R4 batches (S >= 5): 0 = the reference's two formulas bit for bit, 1 = one formula, faster
static int g_i4g_float = 0;     // MOTY_WF_I4G products: 0 = integer path (the reference with IDOT4=1), 1 = f32 x int4 (its default)

// Programmatic dependent launch is on unless the environment says MOTY_CUDA_PDL=0 (read once).
bool moty_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("MOTY_CUDA_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

// ---------------------------------------------------------------------------
// contexts
// ---------------------------------------------------------------------------
static DevCtx g_ctx[MOTY_MAX_DEV];
static int g_nctx = 0;

DevCtx *moty_ctx(int device) {
    for (int i = 0; i < g_nctx; i++)
        if (g_ctx[i].ready && g_ctx[i].dev == device) return &g_ctx[i];
    return nullptr;
}

int moty_grow(DevCtx *c, Buf *b, size_t bytes) {
    if (bytes <= b->cap) return 0;
    if (c->frozen)
        return moty_set_error(MOTY_CUDA_ELIMIT, "scratch of device %d is frozen (moty_cuda_scratch_freeze) and this call needs %zu bytes "
                              "where %zu are reserved: run the largest call before freezing", c->dev, bytes, b->cap);
    MOTY_USE_DEVICE(c->dev);
    if (b->p) { CK(cudaStreamSynchronize(c->stream)); CK(cudaFree(b->p)); b->p = nullptr; b->cap = 0; }
    size_t want = bytes + bytes / 4 + 256;
    CK(cudaMalloc(&b->p, want));
    b->cap = want;
    c->gen++;
    return 0;
}

int moty_grow_pinned(DevCtx *c, Buf *b, size_t bytes) {
    if (bytes <= b->cap) return 0;
    MOTY_USE_DEVICE(c->dev);
    if (b->p) { CK(cudaStreamSynchronize(c->stream)); CK(cudaFreeHost(b->p)); b->p = nullptr; b->cap = 0; }
    size_t want = bytes + bytes / 4 + 256;
    CK(cudaMallocHost(&b->p, want));
    b->cap = want;
    return 0;
}

int moty_grow_zero(DevCtx *c, Buf *b, size_t bytes) {
    if (bytes <= b->cap) return 0;
    CKR(moty_grow(c, b, bytes));
    CK(cudaMemsetAsync(b->p, 0, b->cap, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

static void free_buf(Buf *b) { if (b->p) cudaFree(b->p); b->p = nullptr; b->cap = 0; }
static void free_pinned(Buf *b) { if (b->p) cudaFreeHost(b->p); b->p = nullptr; b->cap = 0; }

extern "C" int moty_cuda_init(const int *devices, int ndev) {
    int zero = 0;
    if (!devices || ndev <= 0) { devices = &zero; ndev = 1; }
    if (ndev > MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "init: %d devices (max %d)", ndev, MOTY_MAX_DEV);
    int have = 0;
    CK(cudaGetDeviceCount(&have));
    for (int i = 0; i < ndev; i++) {
        int d = devices[i];
        if (d < 0 || d >= have) return moty_set_error(MOTY_CUDA_EARG, "init: device %d of %d", d, have);
        if (moty_ctx(d)) continue;
        if (g_nctx >= MOTY_MAX_DEV) return moty_set_error(MOTY_CUDA_EARG, "init: context table full");
        MOTY_USE_DEVICE(d);
        cudaDeviceProp prop;
        CK(cudaGetDeviceProperties(&prop, d));
        if (prop.major != 10)
            return moty_set_error(MOTY_CUDA_EINIT, "device %d is sm_%d%d; this library is built for sm_100a only",
                                  d, prop.major, prop.minor);
        DevCtx *c = &g_ctx[g_nctx];
        *c = DevCtx();
        c->dev = d; c->sms = prop.multiProcessorCount;
        CK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        CK(cudaMalloc(&c->err_dev, 64));
        CK(cudaMemset(c->err_dev, 0, 64));
        CK(cudaMalloc(&c->ctr, 64));
        CK(cudaMemset(c->ctr, 0, 64));
        CK(cudaHostAlloc((void **)&c->hflag, 64, cudaHostAllocMapped | cudaHostAllocPortable));
        c->hflag[0] = 0; c->hseq = 0;
        CK(cudaHostGetDevicePointer((void **)&c->hflag_dev, c->hflag, 0));
        CKR(gemv_q8_init_device());
        CKR(q4r4_init_device());
        c->ready = true;
        g_nctx++;
    }
    return 0;
}

static void host_calls_drop_all();
extern "C" void moty_cuda_shutdown(void) {
    host_calls_drop_all();
    for (int i = 0; i < g_nctx; i++) {
        DevCtx *c = &g_ctx[i];
        if (!c->ready) continue;
        cudaSetDevice(c->dev);
        cudaStreamSynchronize(c->stream);
        Buf *bs[] = {&c->xi, &c->sx, &c->xs, &c->xsum, &c->acc32, &c->dx, &c->dy, &c->dlogits, &c->daux,
                     &c->g, &c->u, &c->h, &c->hq, &c->hs, &c->hxs, &c->hxsum, &c->pair, &c->misc, &c->kcell, &c->rec, &c->mmak, &c->ffn1, &c->attn};
        for (Buf *b : bs) free_buf(b);
        free_pinned(&c->hpin_in); free_pinned(&c->hpin_out);
        if (c->err_dev) cudaFree(c->err_dev);
        if (c->ctr) cudaFree(c->ctr);
        if (c->hflag) cudaFreeHost(c->hflag);
        cudaStreamDestroy(c->stream);
        c->ready = false;
    }
    g_nctx = 0;
}

extern "C" int moty_cuda_sm_count(int device) {
    DevCtx *c = moty_ctx(device);
    return c ? c->sms : moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
}

extern "C" int moty_cuda_sync(int device) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_scratch_freeze(int device, int on) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    c->frozen = on != 0;
    return 0;
}

// ---------------------------------------------------------------------------
// CUDA graphs for callers that do not link the CUDA runtime (a plain-C engine): capture what the *_dev entries enqueue
// on a stream between begin and end, replay it with launch.  The scratch is frozen from begin until the graph is freed
// (it holds the scratch addresses), so the largest call of the captured sequence must have run once before.
// ---------------------------------------------------------------------------
static cudaStream_t pick_stream(DevCtx *c, void *stream) { return stream ? (cudaStream_t)stream : c->stream; }

struct MotyCudaGraph { int device; cudaGraph_t graph; cudaGraphExec_t exec; cudaStream_t stream; bool froze; };

extern "C" int moty_cuda_graph_begin(int device, void *stream) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    cudaStream_t st = pick_stream(c, stream);
    CK(cudaStreamSynchronize(st));
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    return 0;
}

extern "C" int moty_cuda_graph_end(MotyCudaGraph **out, int device, void *stream) {
    if (!out) return moty_set_error(MOTY_CUDA_EARG, "graph_end: null");
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    cudaStream_t st = pick_stream(c, stream);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(st, &g);
    if (e != cudaSuccess || !g) { cudaGetLastError(); return moty_set_error(MOTY_CUDA_ECUDA, "graph_end: capture failed: %s", cudaGetErrorString(e)); }
    cudaGraphExec_t ex = nullptr;
    e = cudaGraphInstantiate(&ex, g, 0);
    if (e != cudaSuccess) { cudaGraphDestroy(g); cudaGetLastError(); return moty_set_error(MOTY_CUDA_ECUDA, "graph_end: instantiate: %s", cudaGetErrorString(e)); }
    MotyCudaGraph *h = new MotyCudaGraph{device, g, ex, st, !c->frozen};
    c->frozen = true;
    *out = h;
    return 0;
}

extern "C" int moty_cuda_graph_launch(MotyCudaGraph *g) {
    if (!g) return moty_set_error(MOTY_CUDA_EARG, "graph_launch: null");
    MOTY_USE_DEVICE(g->device);
    CK(cudaGraphLaunch(g->exec, g->stream));
    return 0;
}

extern "C" int moty_cuda_graph_free(MotyCudaGraph *g) {
    if (!g) return 0;
    DevCtx *c = moty_ctx(g->device);
    if (c) {
        MOTY_USE_DEVICE(g->device);
        cudaStreamSynchronize(g->stream);
        if (g->froze) c->frozen = false;
    }
    cudaGraphExecDestroy(g->exec);
    cudaGraphDestroy(g->graph);
    delete g;
    return 0;
}

extern "C" int moty_cuda_kernel_status(int device, void *stream) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    cudaStream_t st = stream ? (cudaStream_t)stream : c->stream;
    int w[4] = {0, 0, 0, 0};
    CK(cudaMemcpyAsync(w, c->err_dev, 16, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    if (!w[0] && !w[1] && !w[2] && !w[3]) return 0;
    CK(cudaMemsetAsync(c->err_dev, 0, 16, st));
    // a grid barrier that gave up leaves its arrival count and generation inconsistent: back to zero for the next launch
    if (w[1]) CK(cudaMemsetAsync(c->ctr + 4, 0, 8, st));
    CK(cudaStreamSynchronize(st));
    return moty_set_error(MOTY_CUDA_EKERNEL, "kernel error since the last check:%s%s%s%s (results since then are incomplete or wrong)",
                          w[0] ? " tensor-core GEMM pipeline wait expired;" : "", w[1] ? " grid barrier of a one-launch MoE/FFN decode kernel expired;" : "",
                          w[2] ? " bulk-copy wait of a Q4R4/Q8R4 decode kernel expired;" : "",
                          w[3] ? " attention position on the device was outside [0, pos_max] (clamped);" : "");
}

extern "C" int moty_cuda_selftest_expire_wait(int device, int which, void *stream) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    return launch_selftest_expire(which, c->err_dev, reinterpret_cast<unsigned *>(c->ctr) + 4, stream ? (cudaStream_t)stream : c->stream);
}

static cudaStream_t pick_stream(DevCtx *c, void *stream);

extern "C" int moty_cuda_dev_alloc(void **p, size_t bytes, int device) {
    if (!p) return moty_set_error(MOTY_CUDA_EARG, "dev_alloc: null");
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    CK(cudaMalloc(p, bytes ? bytes : 1));
    return 0;
}

extern "C" int moty_cuda_dev_free(void *p) {
    if (p) CK(cudaFree(p));
    return 0;
}

extern "C" int moty_cuda_dev_upload(void *dst_dev, const void *src, size_t bytes, int device, void *stream) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    CK(cudaMemcpyAsync(dst_dev, src, bytes, cudaMemcpyHostToDevice, pick_stream(c, stream)));
    return 0;
}

extern "C" int moty_cuda_dev_download(void *dst, const void *src_dev, size_t bytes, int device, void *stream) {
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    MOTY_USE_DEVICE(device);
    cudaStream_t st = pick_stream(c, stream);
    CK(cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDeviceToHost, st));
    CK(cudaStreamSynchronize(st));
    return 0;
}

extern "C" int moty_cuda_host_alloc(void **p, size_t bytes) {
    if (!p) return moty_set_error(MOTY_CUDA_EARG, "host_alloc: null");
    CK(cudaMallocHost(p, bytes ? bytes : 1));
    return 0;
}

extern "C" int moty_cuda_host_free(void *p) {
    if (p) CK(cudaFreeHost(p));
    return 0;
}


// ---------------------------------------------------------------------------
// weights
// ---------------------------------------------------------------------------
static int mat_sizes(int fmt, int O, int I, size_t *cb, size_t *sb) {
    if (O <= 0 || I <= 0) return moty_set_error(MOTY_CUDA_EARG, "matrix %dx%d", O, I);
    switch (fmt) {
        case MOTY_WF_I8: *cb = (size_t)O * I; *sb = (size_t)O * 4; return 0;
        case MOTY_WF_I4: *cb = (size_t)O * ((I + 1) / 2); *sb = (size_t)O * 4; return 0;
        case MOTY_WF_F32: *cb = (size_t)O * I * 4; *sb = 0; return 0;
        case MOTY_WF_I4G:
            if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "I4G is built for group size 32 and I %% 32 == 0 (I=%d)", I);
            *cb = (size_t)O * (I / 2); *sb = (size_t)O * (I / 32) * 4; return 0;
        case MOTY_WF_Q4R4:
            if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "Q4R4 needs I %% 32 == 0 (I=%d)", I);
            *cb = (size_t)((O + 3) / 4) * (I / 32) * 64; *sb = (size_t)((O + 3) / 4) * (I / 32) * 8; return 0;
        case MOTY_WF_Q8R4:
            if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "Q8R4 needs I %% 32 == 0 (I=%d)", I);
            *cb = (size_t)((O + 3) / 4) * (I / 32) * 128; *sb = (size_t)((O + 3) / 4) * (I / 32) * 8; return 0;
        default: return moty_set_error(MOTY_CUDA_EARG, "unsupported weight format %d", fmt);
    }
}

extern "C" int moty_cuda_upload_mat_rows(MotyCudaMat **out, int fmt, const void *codes, const void *scales,
                                         int O, int I, int o0, int o1, int device) {
    if (!out || !codes) return moty_set_error(MOTY_CUDA_EARG, "upload_mat: null argument");
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    if (o0 < 0 || o1 > O || o0 >= o1) return moty_set_error(MOTY_CUDA_EARG, "upload_mat: rows [%d,%d) of %d", o0, o1, O);
    if (fmt != MOTY_WF_F32 && !scales) return moty_set_error(MOTY_CUDA_EARG, "upload_mat: scales missing");
    if ((fmt == MOTY_WF_Q4R4 || fmt == MOTY_WF_Q8R4) && (o0 % 4))
        return moty_set_error(MOTY_CUDA_EARG, "upload_mat: a Q4R4/Q8R4 shard must start on a block (o0=%d)", o0);
    size_t cb, sb, cb0, sb0;
    int rows = o1 - o0;
    CKR(mat_sizes(fmt, rows, I, &cb, &sb));
    // byte offset of row o0 in the host arrays
    size_t dummy;
    if (o0 > 0) { CKR(mat_sizes(fmt, o0, I, &cb0, &sb0)); } else { cb0 = sb0 = 0; }
    (void)dummy;
    MOTY_USE_DEVICE(device);
    MotyCudaMat *m = new (std::nothrow) MotyCudaMat();
    if (!m) return moty_set_error(MOTY_CUDA_ENOMEM, "upload_mat: host allocation");
    memset(m, 0, sizeof *m);
    m->fmt = fmt; m->O = rows; m->I = I; m->device = device; m->code_bytes = cb; m->scale_bytes = sb;
    if (fmt == MOTY_WF_I4) {
        // Per-row int4 rows are kept as the int8 codes nibble - 8: moty_matmul_i4_s with IDOT4=1 is
        // scale[o] * sx[s] * (float)dot_i4i8(...) (nn/matmul.c:75-101), the integer dot over (nibble - 8) and the Q8_0
        // epilogue, so every Q8_0 kernel -- streaming GEMV, mma.sync batches, tcgen05 GEMM -- serves them bit for bit.
        // Twice the bytes in HBM; a packed-nibble stream for this legacy layout is not built.
        void *packed = nullptr;
        cudaError_t e4 = cudaMalloc(&packed, cb + 256);
        if (e4 == cudaSuccess) e4 = cudaMalloc(&m->codes, (size_t)rows * I + 256);
        if (e4 == cudaSuccess) e4 = cudaMalloc(&m->scales, sb + 256);
        if (e4 == cudaSuccess) e4 = cudaMemcpyAsync(packed, (const char *)codes + cb0, cb, cudaMemcpyHostToDevice, c->stream);
        if (e4 == cudaSuccess) e4 = cudaMemcpyAsync(m->scales, (const char *)scales + sb0, sb, cudaMemcpyHostToDevice, c->stream);
        int rc4 = 0;
        if (e4 == cudaSuccess) rc4 = launch_i4_rows_to_i8((const uint8_t *)packed, (int8_t *)m->codes, rows, I, c->stream);
        if (e4 == cudaSuccess) e4 = cudaStreamSynchronize(c->stream);
        if (packed) cudaFree(packed);
        if (e4 != cudaSuccess || rc4 != 0) {
            if (m->codes) cudaFree(m->codes);
            if (m->scales) cudaFree(m->scales);
            delete m;
            return rc4 != 0 ? rc4 : moty_set_error(MOTY_CUDA_ENOMEM, "upload_mat (int4 rows): %s", cudaGetErrorString(e4));
        }
        m->fmt = MOTY_WF_I8; m->src_fmt = MOTY_WF_I4; m->code_bytes = (size_t)rows * I;
        q8_tc_make_tmap(m);
        *out = m;
        return 0;
    }
    cudaError_t e = cudaMalloc(&m->codes, cb + 256);
    if (e == cudaSuccess && sb) e = cudaMalloc(&m->scales, sb + 256);
    if (e != cudaSuccess) {
        if (m->codes) cudaFree(m->codes);
        delete m;
        return moty_set_error(MOTY_CUDA_ENOMEM, "upload_mat: %s", cudaGetErrorString(e));
    }
    e = cudaMemcpyAsync(m->codes, (const char *)codes + cb0, cb, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess && sb) e = cudaMemcpyAsync(m->scales, (const char *)scales + sb0, sb, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaFree(m->codes); if (m->scales) cudaFree(m->scales); delete m;
        return moty_set_error(MOTY_CUDA_ECUDA, "upload_mat copy: %s", cudaGetErrorString(e));
    }
    if (fmt == MOTY_WF_I8) q8_tc_make_tmap(m);      // optional: absent descriptor = no tensor-core path
    *out = m;
    return 0;
}

extern "C" int moty_cuda_upload_mat(MotyCudaMat **out, int fmt, const void *codes, const void *scales,
                                    int O, int I, int device) {
    return moty_cuda_upload_mat_rows(out, fmt, codes, scales, O, I, 0, O, device);
}

static unsigned long long g_mat_gen = 0;     // bumped when a matrix is freed: its address may come back with other contents
extern "C" int moty_cuda_free_mat(MotyCudaMat *m) {
    if (!m) return 0;
    g_mat_gen++;
    DevCtx *c = moty_ctx(m->device);
    if (c) { cudaSetDevice(m->device); cudaStreamSynchronize(c->stream); }
    if (m->codes) cudaFree(m->codes);
    if (m->scales) cudaFree(m->scales);
    delete m;
    return 0;
}

extern "C" int64_t moty_cuda_mat_bytes(const MotyCudaMat *m) { return m ? (int64_t)(m->code_bytes + m->scale_bytes) : 0; }

extern "C" int moty_cuda_mat_shape(const MotyCudaMat *m, int *fmt, int *O, int *I, int *device) {
    if (!m) return moty_set_error(MOTY_CUDA_EARG, "mat_shape: null");
    if (fmt) *fmt = m->src_fmt ? m->src_fmt : m->fmt;
    if (O) *O = m->O;
    if (I) *I = m->I;
    if (device) *device = m->device;
    return 0;
}

// ---------------------------------------------------------------------------
// mat_apply
// ---------------------------------------------------------------------------
static const int Q8_TC_MIN_S = 9;
// up to this many rows the register-accumulator MMA kernel (weights streamed once) is at least as fast
// as the 128-row tcgen05 tiles; measured crossover on 15360x3840, 151936x1024, 3840x15360
static const int Q8_MMA_MAX_S = 16;

static int mat_apply_on(DevCtx *c, MotyCudaMat *w, float *y, const float *x, int S, int32_t *acc, cudaStream_t st) {
    if (S <= 0) return 0;
    const int I = w->I, O = w->O;
    if (w->fmt == MOTY_WF_F32) return launch_f32_rows((const float *)w->codes, x, y, S, I, O, st);
    if (I > MOTY_QROW_MAX && w->fmt != MOTY_WF_I4G)             // (the grouped int4 layout has its f32 product below)
        return moty_set_error(MOTY_CUDA_ELIMIT, "mat_apply: I=%d exceeds %d (the reference switches to an f32 path there)", I, MOTY_QROW_MAX);
    if (w->fmt == MOTY_WF_I8) {
        // more than 8 rows go to the tensor cores (a 16-token tile, rows past S are zero fill);
        // up to 8 rows stream through the dp4a GEMV
        const bool vec = I % 16 == 0;
        const bool tc = vec && S >= Q8_TC_MIN_S && w->has_tmap && q8_tc_supported(S, I, O);
        const bool stream_ok = vec && !tc && S <= 64;
        if (stream_ok && I > 4096) CKR(moty_grow_zero(c, &c->kcell, (size_t)8 * O * 8));
        if (stream_ok && S == 1 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)
            return launch_q8_stream((const int8_t *)w->codes, (const float *)w->scales, x, nullptr, nullptr, y, acc,
                                    1, I, O, c->ctr, (unsigned long long *)c->kcell.p, c->sms, st);
        CKR(moty_grow(c, &c->xi, (size_t)S * I + 16));
        CKR(moty_grow(c, &c->sx, (size_t)S * 4));
        CKR(launch_qrow_i8(x, (int8_t *)c->xi.p, (float *)c->sx.p, S, I, st));
        // small batches: weights streamed once, mma.sync (split over K when the matrix has few 128-row tiles) -- unless
        // the rows are so long that the tensor-core kernel's split over K does better (3840 x 15360: 29.0 against 31.5 us)
        const bool few_tiles = tc && ((O + 127) / 128) * 4 <= c->sms && I >= 8192;
        if (vec && S > 8 && S <= Q8_MMA_MAX_S && !few_tiles) {
            void *scratch = nullptr;
            if (q8_mma_ksplit(S, I, O, c->sms) > 1) {
                CKR(moty_grow_zero(c, &c->mmak, q8_mma_scratch_bytes(S, O)));
                scratch = c->mmak.p;
            }
            return launch_q8_mma((const int8_t *)w->codes, (const float *)w->scales, (const int8_t *)c->xi.p,
                                 (const float *)c->sx.p, y, acc, S, I, O, scratch, c->sms, st);
        }
        if (tc) return launch_q8_tc(w, (const int8_t *)c->xi.p, (const float *)c->sx.p, y, acc, S, c, st);
        if (stream_ok) {
            for (int s0 = 0; s0 < S; s0 += 8) {
                int ns = S - s0 < 8 ? S - s0 : 8;
                CKR(launch_q8_stream((const int8_t *)w->codes, (const float *)w->scales, nullptr,
                                     (const int8_t *)c->xi.p + (size_t)s0 * I, (const float *)c->sx.p + s0,
                                     y + (size_t)s0 * O, acc ? acc + (size_t)s0 * O : nullptr, ns, I, O, c->ctr,
                                     (unsigned long long *)c->kcell.p, c->sms, st));
            }
            return 0;
        }
        if (!vec)
            return launch_q8_any((const int8_t *)w->codes, (const float *)w->scales, (const int8_t *)c->xi.p,
                                 (const float *)c->sx.p, y, acc, S, I, O, st);
        Q8Args a; memset(&a, 0, sizeof a);
        a.w = (const int8_t *)w->codes; a.scale = (const float *)w->scales;
        a.xi = (const int8_t *)c->xi.p; a.sx = (const float *)c->sx.p;
        a.y = y; a.ldy = O; a.acc = acc; a.S = S; a.I = I; a.O = O;
        return launch_q8_small(a, c->sms, st);
    }
    if (acc) return moty_set_error(MOTY_CUDA_EARG, "int32 accumulators exist for MOTY_WF_I8 only");
    if (w->fmt == MOTY_WF_Q4R4) {
        int nb = I / 32;
        if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "mat_apply: Q4R4 needs I %% 32 == 0");
        if (S == 1 && q4r4_gemv2_supported(I, O, 0, c->sms) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {   // decode, few long rows: two phases
            CKR(moty_grow(c, &c->rec, q4r4_gemv2_scratch_bytes(I, O)));
            return launch_q4r4_gemv2((const uint8_t *)w->codes, (const uint16_t *)w->scales, x, y, (float *)c->rec.p,
                                     c->err_dev + 2, I, O, 0, c->sms, st);
        }
        if (S == 1 && q4r4_gemv_bulk_supported(I, O, c->sms)) {      // decode, a middling row count: quantize once, then stream
            CKR(moty_grow(c, &c->xi, (size_t)I + 16));
            CKR(moty_grow(c, &c->xs, (size_t)nb * 4));
            CKR(moty_grow(c, &c->xsum, (size_t)nb * 4));
            CKR(launch_quant_g32(x, 1, I, (int8_t *)c->xi.p, (float *)c->xs.p, (int32_t *)c->xsum.p, st));
            return launch_q4r4_gemv_bulk((const uint8_t *)w->codes, (const uint16_t *)w->scales, (const int8_t *)c->xi.p,
                                         (const float *)c->xs.p, (const int32_t *)c->xsum.p, y, I, O, c->err_dev + 2,
                                         c->sms, st);
        }
        if (S == 1 && (reinterpret_cast<uintptr_t>(x) & 15) == 0)   // decode: one launch, the row is group-quantized in the kernel
            return launch_q4r4_stream((const uint8_t *)w->codes, (const uint16_t *)w->scales, x, nullptr, nullptr, nullptr,
                                      nullptr, y, 1, I, O, c->sms, st);
        CKR(moty_grow(c, &c->xi, (size_t)S * I + 16));
        CKR(moty_grow(c, &c->xs, (size_t)S * nb * 4));
        CKR(moty_grow(c, &c->xsum, (size_t)S * nb * 4));
        CKR(launch_quant_g32(x, S, I, (int8_t *)c->xi.p, (float *)c->xs.p, (int32_t *)c->xsum.p, st));
        // 2..4 rows: the streaming kernel in one pass for small matrices; on large ones the MMA kernel with one
        // 8-token tile is faster (151936 x 1024 at S = 4: 33 against 44 us, 15360 x 3840: 23 against 32 us)
        if (S <= 4 && (long long)((O + 3) / 4) * nb < 400000) {
            CKR(moty_grow(c, &c->misc, (size_t)S + 16));
            CKR(launch_q4r4_forms((uint8_t *)c->misc.p, S, st));
            return launch_q4r4_stream((const uint8_t *)w->codes, (const uint16_t *)w->scales, nullptr,
                                      (const int8_t *)c->xi.p, (const float *)c->xs.p, (const int32_t *)c->xsum.p,
                                      (const uint8_t *)c->misc.p, y, S, I, O, c->sms, st);
        }
        // batches: integer MMA per group, sequential f32 chain in registers
        CKR(moty_grow(c, &c->rec, (size_t)((S + 7) / 8 * 8) * nb * 16));
        return launch_q4r4_mma((const uint8_t *)w->codes, (const uint16_t *)w->scales, (const int8_t *)c->xi.p,
                               (const float *)c->xs.p, (const int32_t *)c->xsum.p, (int4 *)c->rec.p,
                               y, O, S, I, O, 0, c->sms, st, g_q4r4_relaxed);
    }
    if (w->fmt == MOTY_WF_Q8R4) {
        // the int8 sibling of Q4R4: same group quantizer, same chain, no offset term; one kernel for every S
        const int nb = I / 32;
        if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "mat_apply: Q8R4 needs I %% 32 == 0");
        if (S == 1 && q4r4_gemv2_supported(I, O, 1, c->sms) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {   // decode: two phases
            CKR(moty_grow(c, &c->rec, q4r4_gemv2_scratch_bytes(I, O)));
            return launch_q4r4_gemv2((const uint8_t *)w->codes, (const uint16_t *)w->scales, x, y, (float *)c->rec.p,
                                     c->err_dev + 2, I, O, 1, c->sms, st);
        }
        CKR(moty_grow(c, &c->xi, (size_t)S * I + 16));
        CKR(moty_grow(c, &c->xs, (size_t)S * nb * 4));
        CKR(moty_grow(c, &c->xsum, (size_t)S * nb * 4));
        CKR(moty_grow(c, &c->rec, (size_t)((S + 7) / 8 * 8) * nb * 16));
        CKR(launch_quant_g32(x, S, I, (int8_t *)c->xi.p, (float *)c->xs.p, (int32_t *)c->xsum.p, st));
        return launch_q4r4_mma((const uint8_t *)w->codes, (const uint16_t *)w->scales, (const int8_t *)c->xi.p,
                               (const float *)c->xs.p, (const int32_t *)c->xsum.p, (int4 *)c->rec.p,
                               y, O, S, I, O, 1, c->sms, st, g_q4r4_relaxed);
    }
    if (w->fmt == MOTY_WF_I4G) {
        // moty_matmul_i4_grouped_s: the integer path (IDOT4=1) unless the caller asked for the reference's default, the
        // f32 x int4 product (moty_cuda_set_i4g_float_path); rows the integer path does not take (longer than the
        // quantizer's limit, or not a multiple of 64: nn/matmul.c:172) go to the f32 product there and here
        if (g_i4g_float || I > MOTY_QROW_MAX || (I & 63))
            return launch_i4g_f32_rows((const uint8_t *)w->codes, (const float *)w->scales, x, y, S, I, O, st);
        CKR(moty_grow(c, &c->xi, (size_t)S * I + 16));
        CKR(moty_grow(c, &c->sx, (size_t)S * 4));
        CKR(launch_qrow_i8(x, (int8_t *)c->xi.p, (float *)c->sx.p, S, I, st));
        if (S == 1) {                                           // decode: integer sums in parallel, then the chain
            CKR(moty_grow(c, &c->rec, q4r4_gemv2_scratch_bytes(I, O)));
            return launch_i4g_gemv2((const uint8_t *)w->codes, (const float *)w->scales, (const int8_t *)c->xi.p,
                                    (const float *)c->sx.p, y, (float *)c->rec.p, c->err_dev + 2, I, O, c->sms, st);
        }
        // two rows and more: integer MMA per group, the f32 chain in registers
        CKR(moty_grow(c, &c->rec, i4g_mma_scratch_bytes(S, I)));
        return launch_i4g_mma((const uint8_t *)w->codes, (const float *)w->scales, (const int8_t *)c->xi.p,
                              (const float *)c->sx.p, (int *)c->rec.p, y, S, I, O, c->sms, st);
    }
    return moty_set_error(MOTY_CUDA_EARG, "mat_apply: format %d", w->fmt);
}

extern "C" int moty_cuda_set_i4g_float_path(int on) {
    const int prev = g_i4g_float;
    g_i4g_float = on ? 1 : 0;
    if (prev != g_i4g_float) g_mat_gen++;       // cached graphs of host calls hold the kernels of the other path
    return prev;
}

extern "C" int moty_cuda_set_q4r4_batch_relaxed(int on) {
    const int prev = g_q4r4_relaxed;
    g_q4r4_relaxed = on ? 1 : 0;
    if (prev != g_q4r4_relaxed) g_mat_gen++;
    return prev;
}

extern "C" int moty_cuda_mat_apply_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, int S, void *stream) {
    if (!w || !y_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "mat_apply_dev: null argument");
    DevCtx *c = moty_ctx(w->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", w->device);
    MOTY_USE_DEVICE(w->device);
    return mat_apply_on(c, w, y_dev, x_dev, S, nullptr, pick_stream(c, stream));
}

// One decode row through a MOTY_WF_I8 matrix with the residual add and the RMS norm before it in the same launch:
// y = W * q(rmsnorm(x + t) * g), xout = x + t.  Same bits as add_rmsnorm_dev followed by mat_apply_dev.
extern "C" int moty_cuda_mat_apply_multi_dev(int n, MotyCudaMat *const *w, float *const *y_dev, const float *const *x_dev, void *stream) {
    if (n < 1 || n > 8 || !w || !y_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "mat_apply_multi_dev: n=%d (1..8) or null argument", n);
    const int8_t *codes[8]; const float *scales[8]; int O[8], I[8];
    for (int m = 0; m < n; m++) {
        if (!w[m] || !y_dev[m] || !x_dev[m]) return moty_set_error(MOTY_CUDA_EARG, "mat_apply_multi_dev: null argument for matrix %d", m);
        if (w[m]->fmt != MOTY_WF_I8 || w[m]->device != w[0]->device || !q8_multi_supported(w[m]->I))
            return moty_set_error(MOTY_CUDA_EARG, "mat_apply_multi_dev: matrix %d must be MOTY_WF_I8 on the same GPU with I %% 16 == 0, I <= 16384", m);
        codes[m] = (const int8_t *)w[m]->codes; scales[m] = (const float *)w[m]->scales; O[m] = w[m]->O; I[m] = w[m]->I;
    }
    DevCtx *c = moty_ctx(w[0]->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", w[0]->device);
    MOTY_USE_DEVICE(w[0]->device);
    // rows longer than 4096 values are split in K and meet in 64-bit cells (zero between launches), one run per matrix
    unsigned long long *cells[8] = {nullptr};
    size_t ncell = 0;
    for (int m = 0; m < n; m++) if (I[m] > 4096) ncell += (size_t)O[m];
    if (ncell) {
        CKR(moty_grow_zero(c, &c->kcell, ncell * 8));
        size_t off = 0;
        for (int m = 0; m < n; m++) if (I[m] > 4096) { cells[m] = (unsigned long long *)c->kcell.p + off; off += (size_t)O[m]; }
    }
    return launch_q8_multi(n, codes, scales, x_dev, y_dev, O, I, c->sms, pick_stream(c, stream), cells);
}

extern "C" int moty_cuda_mat_addnorm_supported(const MotyCudaMat *w) {
    return w && w->fmt == MOTY_WF_I8 && w->I % 16 == 0 && w->I <= 4096;
}

// CTA 0 writes xout while every other CTA still reads x and t to form its own copy of the row: xout must not overlap either
static bool resnorm_args_ok(const float *x, const float *t, const float *xout, int I) {
    auto overlaps = [&](const float *a) {
        return reinterpret_cast<uintptr_t>(xout) < reinterpret_cast<uintptr_t>(a + I) &&
               reinterpret_cast<uintptr_t>(a) < reinterpret_cast<uintptr_t>(xout + I);
    };
    return !overlaps(x) && !overlaps(t) && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(t)) & 15) == 0;
}

extern "C" int moty_cuda_mat_apply_resnorm_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, const float *t_dev,
                                               const float *g_t_dev, float *xout_dev, const float *g_x_dev, float eps, void *stream) {
    if (!w || !y_dev || !x_dev || !t_dev || !xout_dev || !g_x_dev)
        return moty_set_error(MOTY_CUDA_EARG, "mat_apply_resnorm_dev: null argument");
    if (!moty_cuda_mat_addnorm_supported(w) || !resnorm_args_ok(x_dev, t_dev, xout_dev, w->I))
        return moty_set_error(MOTY_CUDA_EARG, "mat_apply_resnorm_dev: wants a MOTY_WF_I8 matrix with I <= 4096 (a multiple of 16), x and t "
                              "16-byte aligned, and xout overlapping neither x nor t");
    DevCtx *c = moty_ctx(w->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", w->device);
    MOTY_USE_DEVICE(w->device);
    return launch_q8_stream((const int8_t *)w->codes, (const float *)w->scales, x_dev, nullptr, nullptr, y_dev, nullptr,
                            1, w->I, w->O, c->ctr, (unsigned long long *)c->kcell.p, c->sms, pick_stream(c, stream),
                            t_dev, g_x_dev, xout_dev, eps, g_t_dev);
}

extern "C" int moty_cuda_mat_apply_addnorm_dev(MotyCudaMat *w, float *y_dev, const float *x_dev, const float *t_dev,
                                               float *xout_dev, const float *gain_dev, float eps, void *stream) {
    return moty_cuda_mat_apply_resnorm_dev(w, y_dev, x_dev, t_dev, nullptr, xout_dev, gain_dev, eps, stream);
}

// the device-side address of a page-locked host buffer of `bytes` bytes, 16-byte aligned, or null (pageable memory,
// device memory, an odd alignment, a range that leaves the page-locked allocation)
static void *mapped_alias(const void *p, size_t bytes) {
    cudaPointerAttributes at, end;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (at.type != cudaMemoryTypeHost || !at.devicePointer || (reinterpret_cast<uintptr_t>(at.devicePointer) & 15)) return nullptr;
    if (cudaPointerGetAttributes(&end, (const char *)p + bytes - 1) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    if (end.type != cudaMemoryTypeHost || (const char *)end.devicePointer != (const char *)at.devicePointer + bytes - 1) return nullptr;
    return at.devicePointer;
}
// MOTY_CUDA_HOST_KERNELS=0 in the environment: the host-pointer entries always use copy-engine transfers (read once)
static bool host_kernels_on() {
    static int on = -1;
    if (on < 0) { const char *e = getenv("MOTY_CUDA_HOST_KERNELS"); on = (e && e[0] == '0') ? 0 : 1; }
    return on == 1;
}

// repeated host calls with pinned buffers, replayed as graphs (see mat_apply_host)
struct HostCall { const MotyCudaMat *w; const void *x; void *y; int S, device; unsigned long long gen; cudaGraph_t graph; cudaGraphExec_t exec; };
// an open hash table: a key lives in one of HOST_PROBE slots from its hash on (an engine that serves every matrix of a
// model through one pair of staging buffers has hundreds of live keys)
constexpr int HOST_CALLS = 2048, HOST_PROBE = 8;
static HostCall g_hostcalls_all[MOTY_MAX_DEV][HOST_CALLS];      // one table per device context: calls on different GPUs
static unsigned g_hostcall_next_all[MOTY_MAX_DEV];               // may come from different host threads
static inline unsigned host_call_hash(const MotyCudaMat *w, const void *x, const void *y, int S) {
    unsigned long long h = (reinterpret_cast<uintptr_t>(w) >> 4) * 0x9E3779B97F4A7C15ull;
    h ^= (reinterpret_cast<uintptr_t>(x) >> 4) * 0xC2B2AE3D27D4EB4Full;
    h ^= (reinterpret_cast<uintptr_t>(y) >> 4) * 0x165667B19E3779F9ull;
    h ^= (unsigned long long)S * 0x27D4EB2F165667C5ull;
    return (unsigned)(h >> 40) & (HOST_CALLS - 1);
}
static void host_call_drop(HostCall *h) {
    if (h->exec) cudaGraphExecDestroy(h->exec);
    if (h->graph) cudaGraphDestroy(h->graph);
    *h = HostCall{};
}

static void host_calls_drop_all() {
    for (int d = 0; d < MOTY_MAX_DEV; d++)
        for (int i = 0; i < HOST_CALLS; i++) host_call_drop(&g_hostcalls_all[d][i]);
}

// host-pointer wrapper shared by the entries below: copy in, run, copy out, wait
static int mat_apply_host(MotyCudaMat *w, float *y, int32_t *acc, const float *x, int S) {
    if (!w || !y || !x) return moty_set_error(MOTY_CUDA_EARG, "mat_apply: null argument");
    if (S <= 0) return 0;
    DevCtx *c = moty_ctx(w->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", w->device);
    MOTY_USE_DEVICE(w->device);
    size_t xb = (size_t)S * w->I * 4, yb = (size_t)S * w->O * 4;
    CKR(moty_grow(c, &c->dx, xb));
    if (acc) CKR(moty_grow(c, &c->acc32, yb));
    CKR(moty_grow(c, &c->dy, yb));
    // kernels with bounded waits leave a word behind when one expired: [0] the tensor-core GEMM, [2] the Q4R4 decode
    // kernels fed by bulk copies
    const bool check = S >= Q8_TC_MIN_S || (S == 1 && (w->fmt == MOTY_WF_Q4R4 || w->fmt == MOTY_WF_Q8R4 || w->fmt == MOTY_WF_I4G));
    // Pinned buffers at both ends and nothing else to bring back: kernels move x in and y out, chained to the product, and
    // the host waits for the flag word the last of them writes (hostio.cu) -- no copy-engine transfer, no stream
    // synchronisation.  Anything else (pageable buffers, the accumulator output, kernels with an error word) takes the
    // copies below.
    const float *x_map = nullptr; float *y_map = nullptr;
    if (!acc && !check && host_kernels_on() && (x_map = (const float *)mapped_alias(x, xb)) != nullptr &&
        (y_map = (float *)mapped_alias(y, yb)) != nullptr) {
        const unsigned seq = ++c->hseq;
        unsigned *ctr = reinterpret_cast<unsigned *>(c->ctr) + 8;
        auto enqueue = [&]() -> int {
            CKR(launch_stage_in((float *)c->dx.p, x_map, (long long)S * w->I, c->stream));
            CKR(mat_apply_on(c, w, (float *)c->dy.p, (const float *)c->dx.p, S, nullptr, c->stream));
            return launch_tail_out(y_map, (const float *)c->dy.p, (long long)S * w->O, ctr, c->hflag_dev, c->sms, c->stream);
        };
        // A call that repeats with the same matrix and buffers (a decode loop) is replayed as ONE graph of its three
        // launches: first sight runs it launch by launch, second sight captures it, from then on one submission per call.
        // A graph holds scratch and matrix addresses, so it is only used while neither has moved or been freed since.
        HostCall *hit = nullptr, *slot = nullptr;
        HostCall *g_hostcalls = g_hostcalls_all[c - g_ctx];
        unsigned &g_hostcall_next = g_hostcall_next_all[c - g_ctx];
        const unsigned long long gen = c->gen + g_mat_gen;
        const unsigned h0 = host_call_hash(w, x_map, y_map, S);
        for (int i = 0; i < HOST_PROBE; i++) {
            HostCall *h = &g_hostcalls[(h0 + i) & (HOST_CALLS - 1)];
            if (h->w == w && h->x == x_map && h->y == y_map && h->S == S && h->device == w->device) { hit = h; break; }
            if (!slot && !h->w) slot = h;
        }
        if (hit && hit->gen != gen) { host_call_drop(hit); hit = nullptr; }
        if (hit && hit->exec) {
            CK(cudaGraphLaunch(hit->exec, c->stream));
        } else if (hit) {                                          // second sight: capture (the first run sized every buffer)
            cudaGraph_t g = nullptr;
            CK(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
            const int rc = enqueue();
            const cudaError_t e = cudaStreamEndCapture(c->stream, &g);
            if (rc != 0 || e != cudaSuccess || !g || c->gen + g_mat_gen != gen || cudaGraphInstantiate(&hit->exec, g, 0) != cudaSuccess) {
                cudaGetLastError();
                if (g) cudaGraphDestroy(g);
                hit->exec = nullptr; hit->w = nullptr;             // give up on this key for now
                CKR(enqueue());
            } else {
                hit->graph = g;
                CK(cudaGraphLaunch(hit->exec, c->stream));
            }
        } else {
            if (!hit) {
                if (!slot) { slot = &g_hostcalls[(h0 + g_hostcall_next++ % HOST_PROBE) & (HOST_CALLS - 1)]; host_call_drop(slot); }
                slot->w = w; slot->x = x_map; slot->y = y_map; slot->S = S; slot->device = w->device; slot->gen = gen;
                slot->exec = nullptr; slot->graph = nullptr;
            }
            CKR(enqueue());
        }
        volatile unsigned *flag = c->hflag;
        for (long long spin = 0; *flag != seq; spin++) {
            if (spin >= (1LL << 22) || ((spin & 1023) == 1023 && cudaStreamQuery(c->stream) != cudaErrorNotReady)) {
                // a fraction of a second has passed, or the stream has drained (or failed): let the driver wait and report,
                // then bring the host's count back in step with the device's
                CK(cudaStreamSynchronize(c->stream));
                if (*flag == seq) break;
                unsigned dev_seq = 0;
                CK(cudaMemcpy(&dev_seq, ctr + 1, 4, cudaMemcpyDeviceToHost));
                c->hseq = dev_seq;
                return moty_set_error(MOTY_CUDA_EKERNEL, "mat_apply: the result copy did not report completion");
            }
        }
        return 0;
    }
    CK(cudaMemcpyAsync(c->dx.p, x, xb, cudaMemcpyHostToDevice, c->stream));
    CKR(mat_apply_on(c, w, (float *)c->dy.p, (const float *)c->dx.p, S, acc ? (int32_t *)c->acc32.p : nullptr, c->stream));
    // (letting the GEMV write a pinned result buffer directly, so that the bytes cross PCIe while the weights stream, was
    // measured slower than this copy: 1142 against 1203 GB/s end to end on the six-matrix pass)
    CK(cudaMemcpyAsync(y, c->dy.p, yb, cudaMemcpyDeviceToHost, c->stream));
    if (acc) CK(cudaMemcpyAsync(acc, c->acc32.p, yb, cudaMemcpyDeviceToHost, c->stream));
    int kerr[4] = {0, 0, 0, 0};
    if (check) CK(cudaMemcpyAsync(kerr, c->err_dev, 16, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    if (kerr[0]) {
        cudaMemsetAsync(c->err_dev, 0, 4, c->stream);
        return moty_set_error(MOTY_CUDA_EKERNEL, "tensor-core GEMM gave up on a bounded wait (no result written)");
    }
    if (kerr[2]) {
        cudaMemsetAsync(c->err_dev + 2, 0, 4, c->stream);
        return moty_set_error(MOTY_CUDA_EKERNEL, "Q4R4/Q8R4 decode kernel gave up on a bounded wait (result incomplete)");
    }
    return 0;
}

extern "C" int moty_cuda_mat_apply(MotyCudaMat *w, float *y, const float *x, int S) {
    return mat_apply_host(w, y, nullptr, x, S);
}

extern "C" int moty_cuda_mat_apply_acc(MotyCudaMat *w, float *y, int32_t *acc, const float *x, int S) {
    if (w && w->fmt != MOTY_WF_I8) return moty_set_error(MOTY_CUDA_EARG, "mat_apply_acc: MOTY_WF_I8 only");
    return mat_apply_host(w, y, acc, x, S);
}

static int first_device() {
    for (int i = 0; i < g_nctx; i++) if (g_ctx[i].ready) return g_ctx[i].dev;
    return -1;
}

extern "C" int moty_cuda_matmul_q_s(float *y, const float *x, const int8_t *q, const float *scale, int S, int I, int O) {
    int dev = first_device();
    if (dev < 0) return moty_set_error(MOTY_CUDA_EINIT, "library not initialised");
    MotyCudaMat *m = nullptr;
    CKR(moty_cuda_upload_mat(&m, MOTY_WF_I8, q, scale, O, I, dev));
    int r = moty_cuda_mat_apply(m, y, x, S);
    moty_cuda_free_mat(m);
    return r;
}

extern "C" int moty_cuda_matmul_q8r4_s(float *y, const float *x, const int8_t *q8, const uint16_t *s16, int S, int I, int O) {
    int dev = first_device();
    if (dev < 0) return moty_set_error(MOTY_CUDA_EINIT, "library not initialised");
    MotyCudaMat *m = nullptr;
    CKR(moty_cuda_upload_mat(&m, MOTY_WF_Q8R4, q8, s16, O, I, dev));
    int r = moty_cuda_mat_apply(m, y, x, S);
    moty_cuda_free_mat(m);
    return r;
}

extern "C" int moty_cuda_matmul_i4_grouped_s(float *y, const float *x, const uint8_t *q4, const float *scale,
                                             int S, int I, int O, int gs) {
    int dev = first_device();
    if (dev < 0) return moty_set_error(MOTY_CUDA_EINIT, "library not initialised");
    if (gs != 32) return moty_set_error(MOTY_CUDA_EARG, "matmul_i4_grouped_s: group size 32 only (gs=%d)", gs);
    MotyCudaMat *m = nullptr;
    CKR(moty_cuda_upload_mat(&m, MOTY_WF_I4G, q4, scale, O, I, dev));
    int r = moty_cuda_mat_apply(m, y, x, S);
    moty_cuda_free_mat(m);
    return r;
}

extern "C" int moty_cuda_matmul_q4r4_s(float *y, const float *x, const uint8_t *q4, const uint16_t *s16, int S, int I, int O) {
    int dev = first_device();
    if (dev < 0) return moty_set_error(MOTY_CUDA_EINIT, "library not initialised");
    MotyCudaMat *m = nullptr;
    CKR(moty_cuda_upload_mat(&m, MOTY_WF_Q4R4, q4, s16, O, I, dev));
    int r = moty_cuda_mat_apply(m, y, x, S);
    moty_cuda_free_mat(m);
    return r;
}

// ---------------------------------------------------------------------------
// kernels of the hw.h contract
// ---------------------------------------------------------------------------
static int ctx0(DevCtx **c) {
    int dev = first_device();
    if (dev < 0) return moty_set_error(MOTY_CUDA_EINIT, "library not initialised");
    *c = moty_ctx(dev);
    MOTY_USE_DEVICE(dev);
    return 0;
}

// The *_dev entries that take no matrix or layer handle run on the GPU that OWNS their first device pointer
// (a process may have initialised several GPUs; the first one is only the default of the host-pointer entries).
static int ctx_of(const void *dev_ptr, DevCtx **c) {
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, dev_ptr);
    if (e != cudaSuccess || (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged)) {
        (void)cudaGetLastError();
        return moty_set_error(MOTY_CUDA_EARG, "not a device pointer");
    }
    *c = moty_ctx(at.device);
    if (!*c) return moty_set_error(MOTY_CUDA_EINIT, "device %d (owner of the pointer) not initialised", at.device);
    return 0;
}
// the context of the GPU that owns dev_ptr, and that GPU current until the end of the caller's scope
#define MOTY_CTX_OF(dev_ptr, c) DevCtx *c; CKR(ctx_of(dev_ptr, &c)); MOTY_USE_DEVICE(c->dev)

extern "C" int moty_cuda_qrow_i8_dev(const float *x_dev, int8_t *q_dev, float *scale_dev, int rows, int n, void *stream) {
    MOTY_CTX_OF(x_dev, c);
    return launch_qrow_i8(x_dev, q_dev, scale_dev, rows, n, pick_stream(c, stream));
}

extern "C" int moty_cuda_qrow_i8(const float *x, int8_t *q, float *scale, int rows, int n) {
    DevCtx *c; CKR(ctx0(&c));
    if (rows <= 0 || n <= 0) return 0;
    size_t nb = (size_t)rows * n;
    CKR(moty_grow(c, &c->dx, nb * 4));
    CKR(moty_grow(c, &c->xi, nb + 16));
    CKR(moty_grow(c, &c->sx, (size_t)rows * 4));
    CK(cudaMemcpyAsync(c->dx.p, x, nb * 4, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_qrow_i8((const float *)c->dx.p, (int8_t *)c->xi.p, (float *)c->sx.p, rows, n, c->stream));
    CK(cudaMemcpyAsync(q, c->xi.p, nb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(scale, c->sx.p, (size_t)rows * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_quant_g32_dev(const float *x_dev, int rows, int I, int8_t *xq_dev, float *xs_dev,
                                       int32_t *xsum_dev, void *stream) {
    MOTY_CTX_OF(x_dev, c);
    if (I % 32) return moty_set_error(MOTY_CUDA_EARG, "quant_g32: I=%d", I);
    return launch_quant_g32(x_dev, rows, I, xq_dev, xs_dev, xsum_dev, pick_stream(c, stream));
}

extern "C" int moty_cuda_quant_g32(const float *x, int rows, int I, int8_t *xq, float *xs, int32_t *xsum) {
    DevCtx *c; CKR(ctx0(&c));
    if (I % 32 || I <= 0) return moty_set_error(MOTY_CUDA_EARG, "quant_g32: I=%d", I);
    if (rows <= 0) return 0;
    size_t n = (size_t)rows * I, ng = (size_t)rows * (I / 32);
    CKR(moty_grow(c, &c->dx, n * 4));
    CKR(moty_grow(c, &c->xi, n + 16));
    CKR(moty_grow(c, &c->xs, ng * 4));
    CKR(moty_grow(c, &c->xsum, ng * 4));
    CK(cudaMemcpyAsync(c->dx.p, x, n * 4, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_quant_g32((const float *)c->dx.p, rows, I, (int8_t *)c->xi.p, (float *)c->xs.p, (int32_t *)c->xsum.p, c->stream));
    CK(cudaMemcpyAsync(xq, c->xi.p, n, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(xs, c->xs.p, ng * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(xsum, c->xsum.p, ng * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

static int dot_rows_host(const void *w, size_t wbytes, const int8_t *x, int nrows, int n, int32_t *out, int i4) {
    DevCtx *c; CKR(ctx0(&c));
    if (nrows <= 0) return 0;
    if (n < 0) return moty_set_error(MOTY_CUDA_EARG, "dot: n=%d", n);
    CKR(moty_grow(c, &c->dx, wbytes + 16));
    CKR(moty_grow(c, &c->xi, (size_t)n + 16));
    CKR(moty_grow(c, &c->acc32, (size_t)nrows * 4));
    if (wbytes) CK(cudaMemcpyAsync(c->dx.p, w, wbytes, cudaMemcpyHostToDevice, c->stream));
    if (n) CK(cudaMemcpyAsync(c->xi.p, x, n, cudaMemcpyHostToDevice, c->stream));
    if (i4) CKR(launch_dot_i4i8_rows((const uint8_t *)c->dx.p, (const int8_t *)c->xi.p, nrows, n, (int32_t *)c->acc32.p, c->stream));
    else CKR(launch_dot_i8i8_rows((const int8_t *)c->dx.p, (const int8_t *)c->xi.p, nrows, n, (int32_t *)c->acc32.p, c->stream));
    CK(cudaMemcpyAsync(out, c->acc32.p, (size_t)nrows * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_dot_i8i8(const int8_t *w, const int8_t *x, int nrows, int n, int32_t *out) {
    return dot_rows_host(w, (size_t)nrows * n, x, nrows, n, out, 0);
}

extern "C" int moty_cuda_dot_i4i8(const uint8_t *w4, const int8_t *x, int nrows, int n, int32_t *out) {
    return dot_rows_host(w4, (size_t)nrows * ((n + 1) / 2), x, nrows, n, out, 1);
}

// ---------------------------------------------------------------------------
// router
// ---------------------------------------------------------------------------
static int route_host(const float *in, int rows, int E, int K, int *idx, float *w, float *probs_out, int softmax, int norm) {
    DevCtx *c; CKR(ctx0(&c));
    if (rows <= 0) return 0;
    size_t lb = (size_t)rows * E * 4, kb = (size_t)rows * K * 4;
    CKR(moty_grow(c, &c->dlogits, lb));
    CKR(moty_grow(c, &c->daux, lb + 2 * kb));
    float *probs = (float *)c->daux.p;
    int *didx = (int *)((char *)c->daux.p + lb);
    float *dw = (float *)((char *)c->daux.p + lb + kb);
    CK(cudaMemcpyAsync(c->dlogits.p, in, lb, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_route((const float *)c->dlogits.p, rows, E, K, didx, dw, probs_out ? probs : nullptr, softmax, norm, c->stream));
    CK(cudaMemcpyAsync(idx, didx, kb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(w, dw, kb, cudaMemcpyDeviceToHost, c->stream));
    if (probs_out) CK(cudaMemcpyAsync(probs_out, probs, lb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_moe_topk(const float *probs, int rows, int E, int K, int *idx, float *w, int norm_topk) {
    return route_host(probs, rows, E, K, idx, w, nullptr, 0, norm_topk);
}

extern "C" int moty_cuda_route_topk(const float *logits, int rows, int E, int K, int *idx, float *w, float *probs_out) {
    return route_host(logits, rows, E, K, idx, w, probs_out, 1, 1);
}

extern "C" int moty_cuda_route_topk_dev(const float *logits_dev, int rows, int E, int K, int *idx_dev, float *w_dev,
                                        float *probs_dev, int norm_topk, void *stream) {
    MOTY_CTX_OF(logits_dev, c);
    return launch_route(logits_dev, rows, E, K, idx_dev, w_dev, probs_dev, 1, norm_topk, pick_stream(c, stream));
}

// ---------------------------------------------------------------------------
// greedy token
// ---------------------------------------------------------------------------
extern "C" int moty_cuda_argmax_dev(const float *v_dev, int n, int *out_dev, void *stream) {
    MOTY_CTX_OF(v_dev, c);
    CKR(moty_grow(c, &c->daux, 4096));
    return launch_argmax_scratch(v_dev, n, out_dev, (float *)c->daux.p, (int *)((char *)c->daux.p + 1024),
                                 pick_stream(c, stream));
}

extern "C" int moty_cuda_argmax(const float *v, int n, int *out) {
    DevCtx *c; CKR(ctx0(&c));
    if (n <= 0 || !v || !out) return moty_set_error(MOTY_CUDA_EARG, "argmax: n=%d", n);
    CKR(moty_grow(c, &c->dx, (size_t)n * 4));
    CKR(moty_grow(c, &c->daux, 4096));
    CK(cudaMemcpyAsync(c->dx.p, v, (size_t)n * 4, cudaMemcpyHostToDevice, c->stream));
    int *dout = (int *)((char *)c->daux.p + 2048);
    CKR(launch_argmax_scratch((const float *)c->dx.p, n, dout, (float *)c->daux.p, (int *)((char *)c->daux.p + 1024), c->stream));
    CK(cudaMemcpyAsync(out, dout, 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// lm_head + greedy token in one call: the logits stay on the device, one int per row comes back
extern "C" int moty_cuda_head_argmax_dev(MotyCudaMat *head, const float *x_dev, int S, int *ids_dev, float *logits_dev,
                                         void *stream) {
    if (!head || !x_dev || !ids_dev) return moty_set_error(MOTY_CUDA_EARG, "head_argmax_dev: null argument");
    if (S <= 0) return 0;
    DevCtx *c = moty_ctx(head->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", head->device);
    MOTY_USE_DEVICE(head->device);
    cudaStream_t st = pick_stream(c, stream);
    float *lg = logits_dev;
    if (!lg) {
        CKR(moty_grow(c, &c->dlogits, (size_t)S * head->O * 4));
        lg = (float *)c->dlogits.p;
    }
    CKR(moty_grow(c, &c->daux, 4096));
    CKR(mat_apply_on(c, head, lg, x_dev, S, nullptr, st));
    for (int s = 0; s < S; s++)
        CKR(launch_argmax_scratch(lg + (size_t)s * head->O, head->O, ids_dev + s, (float *)c->daux.p,
                                  (int *)((char *)c->daux.p + 1024), st));
    return 0;
}

extern "C" int moty_cuda_head_argmax(MotyCudaMat *head, const float *x, int S, int *ids, float *logits) {
    if (!head || !x || !ids) return moty_set_error(MOTY_CUDA_EARG, "head_argmax: null argument");
    if (S <= 0) return 0;
    DevCtx *c = moty_ctx(head->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", head->device);
    MOTY_USE_DEVICE(head->device);
    const size_t xb = (size_t)S * head->I * 4, lb = (size_t)S * head->O * 4;
    CKR(moty_grow(c, &c->dx, xb));
    CKR(moty_grow(c, &c->dlogits, lb));
    CKR(moty_grow(c, &c->daux, 4096 + (size_t)S * 4));
    int *dids = (int *)((char *)c->daux.p + 4096);
    CK(cudaMemcpyAsync(c->dx.p, x, xb, cudaMemcpyHostToDevice, c->stream));
    CKR(moty_cuda_head_argmax_dev(head, (const float *)c->dx.p, S, dids, (float *)c->dlogits.p, c->stream));
    CK(cudaMemcpyAsync(ids, dids, (size_t)S * 4, cudaMemcpyDeviceToHost, c->stream));
    if (logits) CK(cudaMemcpyAsync(logits, c->dlogits.p, lb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// ---------------------------------------------------------------------------
// the f32 steps of a decoder layer around the matmuls (device pointers; they run on the GPU that owns `x_dev`)
// ---------------------------------------------------------------------------
extern "C" int moty_cuda_rmsnorm_dev(float *out_dev, const float *x_dev, const float *w_dev, int S, int D, float eps, void *stream) {
    if (!out_dev || !x_dev || !w_dev) return moty_set_error(MOTY_CUDA_EARG, "rmsnorm_dev: null argument");
    MOTY_CTX_OF(x_dev, c);
    return launch_rmsnorm_rows(out_dev, x_dev, w_dev, S, D, eps, pick_stream(c, stream));
}

extern "C" int moty_cuda_add_dev(float *y_dev, const float *x_dev, long long n, void *stream) {
    if (!y_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "add_dev: null argument");
    MOTY_CTX_OF(x_dev, c);
    return launch_add(y_dev, x_dev, n, pick_stream(c, stream));
}

extern "C" int moty_cuda_add_rmsnorm_dev(float *x_dev, const float *t_dev, float *out_dev, const float *w_dev, int S, int D,
                                         float eps, void *stream) {
    if (!x_dev || !t_dev || !out_dev || !w_dev) return moty_set_error(MOTY_CUDA_EARG, "add_rmsnorm_dev: null argument");
    MOTY_CTX_OF(x_dev, c);
    return launch_add_rmsnorm_rows(x_dev, t_dev, out_dev, w_dev, S, D, eps, pick_stream(c, stream));
}

extern "C" int moty_cuda_normadd_rmsnorm_dev(float *x_dev, const float *t_dev, const float *g_t_dev, float *out_dev, const float *g_x_dev,
                                             int S, int D, float eps, void *stream) {
    if (!x_dev || !t_dev || !g_t_dev || (out_dev && !g_x_dev)) return moty_set_error(MOTY_CUDA_EARG, "normadd_rmsnorm_dev: null argument");
    MOTY_CTX_OF(x_dev, c);
    return launch_normadd_rmsnorm_rows(x_dev, t_dev, g_t_dev, out_dev, g_x_dev, S, D, eps, pick_stream(c, stream));
}

extern "C" int moty_cuda_embed_rows_dev(MotyCudaMat *embed, float *out_dev, const int *ids_dev, int S, float scale, void *stream) {
    if (!embed || !out_dev || !ids_dev) return moty_set_error(MOTY_CUDA_EARG, "embed_rows_dev: null argument");
    if (embed->fmt != MOTY_WF_I8) return moty_set_error(MOTY_CUDA_EARG, "embed_rows_dev: MOTY_WF_I8 table only");
    DevCtx *c = moty_ctx(embed->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", embed->device);
    MOTY_USE_DEVICE(embed->device);
    return launch_embed_rows(out_dev, (const int8_t *)embed->codes, (const float *)embed->scales, ids_dev, S, embed->I, embed->O,
                             scale, pick_stream(c, stream));
}

// ---------------------------------------------------------------------------
// attention core of one layer (KV cache resident on the device)
// ---------------------------------------------------------------------------
struct MotyCudaAttn {
    int H, KV, hd, rot, max_t, kv8, device;
    float theta, eps;
    int gemma, window; float scale;      // engines/gemma.c's attention: p-RoPE pairs, sliding window, given score scale
    float *qn, *kn, *vn;
    float *K, *V; int8_t *K8, *V8; float *Ks, *Vs;
};

extern "C" int moty_cuda_attn_free(MotyCudaAttn *a) {
    if (!a) return 0;
    DevCtx *c = moty_ctx(a->device);
    if (c) { cudaSetDevice(a->device); cudaStreamSynchronize(c->stream); }
    void *ps[] = {a->qn, a->kn, a->vn, a->K, a->V, a->K8, a->V8, a->Ks, a->Vs};
    for (void *p : ps) if (p) cudaFree(p);
    delete a;
    return 0;
}

extern "C" int moty_cuda_attn_create(MotyCudaAttn **out, int n_heads, int n_kv_heads, int head_dim, int rot, float theta,
                                     float eps, const float *qn, const float *kn, int max_t, int kv8, int device) {
    if (!out) return moty_set_error(MOTY_CUDA_EARG, "attn_create: null argument");
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || head_dim <= 0 || head_dim > 256 || rot < 0 ||
        rot > head_dim || (rot & 1) || max_t <= 0)
        return moty_set_error(MOTY_CUDA_EARG, "attn_create: H=%d KV=%d hd=%d rot=%d max_t=%d", n_heads, n_kv_heads, head_dim, rot, max_t);
    MOTY_USE_DEVICE(device);
    MotyCudaAttn *a = new (std::nothrow) MotyCudaAttn();
    if (!a) return moty_set_error(MOTY_CUDA_ENOMEM, "attn_create: host allocation");
    memset(a, 0, sizeof *a);
    a->H = n_heads; a->KV = n_kv_heads; a->hd = head_dim; a->rot = rot; a->max_t = max_t; a->kv8 = kv8 ? 1 : 0;
    a->device = device; a->theta = theta; a->eps = eps;
    const size_t rows = (size_t)n_kv_heads * max_t;
    cudaError_t e = cudaSuccess;
    if (qn) e = cudaMalloc(&a->qn, (size_t)head_dim * 4);
    if (e == cudaSuccess && kn) e = cudaMalloc(&a->kn, (size_t)head_dim * 4);
    if (e == cudaSuccess && a->kv8) {
        e = cudaMalloc(&a->K8, rows * head_dim);
        if (e == cudaSuccess) e = cudaMalloc(&a->V8, rows * head_dim);
        if (e == cudaSuccess) e = cudaMalloc(&a->Ks, rows * 4);
        if (e == cudaSuccess) e = cudaMalloc(&a->Vs, rows * 4);
    } else if (e == cudaSuccess) {
        e = cudaMalloc(&a->K, rows * head_dim * 4);
        if (e == cudaSuccess) e = cudaMalloc(&a->V, rows * head_dim * 4);
    }
    // positions never written read as zero rows (score 0, value 0), the same on every run
    if (e == cudaSuccess && a->kv8) {
        e = cudaMemsetAsync(a->K8, 0, rows * head_dim, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(a->V8, 0, rows * head_dim, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(a->Ks, 0, rows * 4, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(a->Vs, 0, rows * 4, c->stream);
    } else if (e == cudaSuccess) {
        e = cudaMemsetAsync(a->K, 0, rows * head_dim * 4, c->stream);
        if (e == cudaSuccess) e = cudaMemsetAsync(a->V, 0, rows * head_dim * 4, c->stream);
    }
    if (e == cudaSuccess && qn) e = cudaMemcpyAsync(a->qn, qn, (size_t)head_dim * 4, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess && kn) e = cudaMemcpyAsync(a->kn, kn, (size_t)head_dim * 4, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        moty_cuda_attn_free(a);
        return moty_set_error(MOTY_CUDA_ENOMEM, "attn_create: %s", cudaGetErrorString(e));
    }
    *out = a;
    return 0;
}

extern "C" int moty_cuda_attn_create_gemma(MotyCudaAttn **out, int n_heads, int n_kv_heads, int head_dim, int rot_pairs, float theta,
                                           float eps, const float *qn, const float *kn, const float *vn, int window, float scale,
                                           int max_t, int kv8, int device) {
    if (rot_pairs < 0 || rot_pairs > head_dim / 2 || (head_dim & 1) || window < 0 || scale < 0.f)
        return moty_set_error(MOTY_CUDA_EARG, "attn_create_gemma: hd=%d rot_pairs=%d window=%d scale=%g", head_dim, rot_pairs, window, (double)scale);
    MotyCudaAttn *a = nullptr;
    CKR(moty_cuda_attn_create(&a, n_heads, n_kv_heads, head_dim, 0, theta, eps, qn, kn, max_t, kv8, device));
    a->gemma = 1; a->rot = rot_pairs; a->window = window; a->scale = scale;
    if (vn) {
        DevCtx *c = moty_ctx(device);
        MOTY_USE_DEVICE(device);
        cudaError_t e = cudaMalloc(&a->vn, (size_t)head_dim * 4);
        if (e == cudaSuccess) e = cudaMemcpyAsync(a->vn, vn, (size_t)head_dim * 4, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (e != cudaSuccess) { moty_cuda_attn_free(a); return moty_set_error(MOTY_CUDA_ENOMEM, "attn_create_gemma: %s", cudaGetErrorString(e)); }
    }
    *out = a;
    return 0;
}

static int attn_core_on(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev, int S, int pos_base,
                        const int *pos_dev, void *stream);

extern "C" int moty_cuda_attn_core_dev(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev,
                                       int S, int pos_base, void *stream) {
    return attn_core_on(a, ctx_dev, q_dev, k_dev, v_dev, S, pos_base, nullptr, stream);
}

extern "C" int moty_cuda_attn_core_posdev(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev,
                                          int S, const int *pos_dev, int pos_max, void *stream) {
    if (!pos_dev) return moty_set_error(MOTY_CUDA_EARG, "attn_core_posdev: null position");
    return attn_core_on(a, ctx_dev, q_dev, k_dev, v_dev, S, pos_max, pos_dev, stream);
}

static int attn_core_on(MotyCudaAttn *a, float *ctx_dev, float *q_dev, float *k_dev, const float *v_dev, int S, int pos_base,
                        const int *pos_dev, void *stream) {
    if (!a || !ctx_dev || !q_dev || !k_dev || !v_dev) return moty_set_error(MOTY_CUDA_EARG, "attn_core_dev: null argument");
    DevCtx *c = moty_ctx(a->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", a->device);
    MOTY_USE_DEVICE(a->device);
    const size_t sb = attn_scratch_bytes(S, a->H, a->KV, a->hd, c->sms);
    if (sb) CKR(moty_grow(c, &c->attn, sb));
    return launch_attn_core(ctx_dev, q_dev, k_dev, v_dev, S, pos_base, a->H, a->KV, a->hd, a->rot, a->theta, a->eps, a->qn,
                            a->kn, a->K, a->V, a->K8, a->V8, a->Ks, a->Vs, a->max_t, sb ? (float *)c->attn.p : nullptr,
                            pos_dev, c->err_dev + 3, c->sms, pick_stream(c, stream), a->gemma, a->window, a->scale, a->vn);
}

extern "C" int moty_cuda_attn_gate_dev(MotyCudaAttn *a, float *ctx_dev, const float *gate_dev, int S, void *stream) {
    if (!a || !ctx_dev || !gate_dev) return moty_set_error(MOTY_CUDA_EARG, "attn_gate_dev: null argument");
    DevCtx *c = moty_ctx(a->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", a->device);
    MOTY_USE_DEVICE(a->device);
    return launch_attn_gate(ctx_dev, gate_dev, (long long)S * a->H * a->hd, pick_stream(c, stream));
}

extern "C" int moty_cuda_attn_core(MotyCudaAttn *a, float *ctx, const float *q, const float *k, const float *v, int S,
                                   int pos_base) {
    if (!a || !ctx || !q || !k || !v) return moty_set_error(MOTY_CUDA_EARG, "attn_core: null argument");
    if (S <= 0) return 0;
    DevCtx *c = moty_ctx(a->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", a->device);
    MOTY_USE_DEVICE(a->device);
    const size_t qb = (size_t)S * a->H * a->hd * 4, kb = (size_t)S * a->KV * a->hd * 4;
    CKR(moty_grow(c, &c->dx, qb + 2 * kb));
    CKR(moty_grow(c, &c->dy, qb));
    float *dq = (float *)c->dx.p, *dk = (float *)((char *)c->dx.p + qb), *dv = (float *)((char *)c->dx.p + qb + kb);
    CK(cudaMemcpyAsync(dq, q, qb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(dk, k, kb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(dv, v, kb, cudaMemcpyHostToDevice, c->stream));
    CKR(moty_cuda_attn_core_dev(a, (float *)c->dy.p, dq, dk, dv, S, pos_base, c->stream));
    CK(cudaMemcpyAsync(ctx, c->dy.p, qb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// ---------------------------------------------------------------------------
// load-time quantizers
// ---------------------------------------------------------------------------
extern "C" int moty_cuda_quantize_rows(const float *w, int8_t *q, float *scale, int O, int I) {
    DevCtx *c; CKR(ctx0(&c));
    if (O <= 0 || I <= 0) return moty_set_error(MOTY_CUDA_EARG, "quantize_rows: %dx%d", O, I);
    size_t n = (size_t)O * I;
    CKR(moty_grow(c, &c->dx, n * 4));
    CKR(moty_grow(c, &c->dy, n + 16));
    CKR(moty_grow(c, &c->sx, (size_t)O * 4));
    CK(cudaMemcpyAsync(c->dx.p, w, n * 4, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_quantize_rows((const float *)c->dx.p, (int8_t *)c->dy.p, (float *)c->sx.p, O, I, c->stream));
    CK(cudaMemcpyAsync(q, c->dy.p, n, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(scale, c->sx.p, (size_t)O * 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_pack_q4r4(const float *w, int O, int I, uint8_t *q4, uint16_t *s16) {
    DevCtx *c; CKR(ctx0(&c));
    if (O <= 0 || I <= 0 || I % 32) return moty_set_error(MOTY_CUDA_EARG, "pack_q4r4: %dx%d", O, I);
    size_t n = (size_t)O * I, cb, sb;
    CKR(mat_sizes(MOTY_WF_Q4R4, O, I, &cb, &sb));
    CKR(moty_grow(c, &c->dx, n * 4));
    CKR(moty_grow(c, &c->dy, cb + 16));
    CKR(moty_grow(c, &c->daux, sb + 16));
    CK(cudaMemcpyAsync(c->dx.p, w, n * 4, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_pack_q4r4((const float *)c->dx.p, O, I, (uint8_t *)c->dy.p, (uint16_t *)c->daux.p, c->stream));
    CK(cudaMemcpyAsync(q4, c->dy.p, cb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaMemcpyAsync(s16, c->daux.p, sb, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// ---------------------------------------------------------------------------
// dense FFN
// ---------------------------------------------------------------------------
static int g_moe_fast = 1;      // 1: best decode paths; 2: the split decode path; 3: as 1, dense FFN in the cooperative kernel; 0: general path only
static inline bool moe_fast_one() { return g_moe_fast == 1 || g_moe_fast == 3; }
static int g_moe_tc = 1;        // int8 batches: 1 = grouped products on tcgen05 where the experts see >= 8 rows each; 0 = mma.sync tiles

static int ffn_on(DevCtx *c, MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act,
                  float *out, const float *x, int S, cudaStream_t st) {
    int I = gate->O, D = gate->I;
    if (up->O != I || up->I != D || down->O != D || down->I != I)
        return moty_set_error(MOTY_CUDA_EARG, "ffn: shapes gate %dx%d up %dx%d down %dx%d", gate->O, gate->I, up->O, up->I, down->O, down->I);
    if (gate->device != up->device || gate->device != down->device) return moty_set_error(MOTY_CUDA_EARG, "ffn: matrices on different devices");
    if (act != MOTY_ACT_SILU && act != MOTY_ACT_GELU_TANH) return moty_set_error(MOTY_CUDA_EARG, "ffn: activation %d", act);
    size_t hb = (size_t)S * I * 4;
    CKR(moty_grow(c, &c->g, hb));
    // One token, int8 gate and up with rows of at most 4096 values: gate, up and the activation in one launch, then the
    // down product, both chained to their neighbours by programmatic dependent launch.  Same bits as the four steps below.
    // (Measured against the one-launch cooperative kernel further down: 9.6 against 12.0 us for the 1024/3072 block, 9.9
    // against 12.3 us for 2048/4096, 1406 against 1257 tok/s over a whole Qwen3-0.6B-shaped decode -- a cooperative launch
    // cannot be chained, so it pays its whole launch latency and the next kernel's as well.)
    if (S == 1 && (g_moe_fast == 1 || g_moe_fast == 2) && gate->fmt == MOTY_WF_I8 && up->fmt == MOTY_WF_I8 && q8_gateup_supported(I, D) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        CKR(launch_q8_gateup((const int8_t *)gate->codes, (const float *)gate->scales, (const int8_t *)up->codes, (const float *)up->scales,
                             x, (float *)c->g.p, I, D, act, c->sms, st));
        return mat_apply_on(c, down, out, (const float *)c->g.p, S, nullptr, st);
    }
    // Kept as a cross-check (set_moe_fast_path(3)): with int8 matrices and SiLU the block is the MoE decode block with one
    // expert of weight 1 (softmax of a single logit is exp(0)/exp(0) = 1 and 1 * h = h exactly), so the one-launch
    // cooperative kernel takes it: gate/up rows, a grid barrier, the down rows -- same quantizers, same (scale * sx) * acc,
    // same SiLU expression as the steps below.
    if (S == 1 && act == MOTY_ACT_SILU && g_moe_fast == 3 && gate->fmt == MOTY_WF_I8 && up->fmt == MOTY_WF_I8 &&
        down->fmt == MOTY_WF_I8 && moe_decode_fused_q8_supported(1, 1, I, D) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        CKR(moty_grow_zero(c, &c->ffn1, 64));               // [0] the single logit (0), [4] index out, [8] weight out
        char *z = (char *)c->ffn1.p;
        return launch_moe_decode_fused_q8((const float *)z, 1, 0, (int *)(z + 16), (float *)(z + 32),
                                          (const int8_t *)gate->codes, (const int8_t *)up->codes, (const int8_t *)down->codes,
                                          (const float *)gate->scales, (const float *)up->scales, (const float *)down->scales,
                                          0, 0, 0, 0, x, (float *)c->g.p, out, nullptr, 1, I, D, 0, 1,
                                          reinterpret_cast<unsigned *>(c->ctr) + 4, c->err_dev + 1, c->sms, st);
    }
    CKR(moty_grow(c, &c->u, hb));
    CKR(mat_apply_on(c, gate, (float *)c->g.p, x, S, nullptr, st));
    CKR(mat_apply_on(c, up, (float *)c->u.p, x, S, nullptr, st));
    CKR(launch_act_mul((float *)c->g.p, (const float *)c->u.p, (int64_t)S * I, act, st));
    return mat_apply_on(c, down, out, (const float *)c->g.p, S, nullptr, st);
}

extern "C" int moty_cuda_ffn_dev(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act,
                                 float *out_dev, const float *x_dev, int S, void *stream) {
    if (!gate || !up || !down || !out_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "ffn_dev: null argument");
    DevCtx *c = moty_ctx(gate->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", gate->device);
    MOTY_USE_DEVICE(gate->device);
    if (S <= 0) return 0;
    return ffn_on(c, gate, up, down, act, out_dev, x_dev, S, pick_stream(c, stream));
}

extern "C" int moty_cuda_ffn_resnorm_supported(const MotyCudaMat *gate, const MotyCudaMat *up) {
    return gate && up && gate->fmt == MOTY_WF_I8 && up->fmt == MOTY_WF_I8 && gate->O == up->O && gate->I == up->I &&
           q8_gateup_supported(gate->O, gate->I);
}

extern "C" int moty_cuda_ffn_resnorm_dev(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act, float *out_dev,
                                         const float *x_dev, const float *t_dev, const float *g_t_dev, float *xout_dev,
                                         const float *g_x_dev, float eps, void *stream) {
    if (!gate || !up || !down || !out_dev || !x_dev || !t_dev || !xout_dev || !g_x_dev)
        return moty_set_error(MOTY_CUDA_EARG, "ffn_resnorm_dev: null argument");
    if (!moty_cuda_ffn_resnorm_supported(gate, up) || down->O != gate->I || down->I != gate->O || !resnorm_args_ok(x_dev, t_dev, xout_dev, gate->I))
        return moty_set_error(MOTY_CUDA_EARG, "ffn_resnorm_dev: wants MOTY_WF_I8 gate and up [I][D] with D <= 4096 (a multiple of 16), down [D][I], "
                              "x and t 16-byte aligned, and xout overlapping neither x nor t");
    if (gate->device != up->device || gate->device != down->device) return moty_set_error(MOTY_CUDA_EARG, "ffn_resnorm_dev: matrices on different devices");
    if (act != MOTY_ACT_SILU && act != MOTY_ACT_GELU_TANH) return moty_set_error(MOTY_CUDA_EARG, "ffn_resnorm_dev: activation %d", act);
    DevCtx *c = moty_ctx(gate->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", gate->device);
    MOTY_USE_DEVICE(gate->device);
    cudaStream_t st = pick_stream(c, stream);
    const int I = gate->O, D = gate->I;
    CKR(moty_grow(c, &c->g, (size_t)I * 4));
    CKR(launch_q8_gateup((const int8_t *)gate->codes, (const float *)gate->scales, (const int8_t *)up->codes, (const float *)up->scales,
                         x_dev, (float *)c->g.p, I, D, act, c->sms, st, t_dev, g_t_dev, g_x_dev, xout_dev, eps));
    return mat_apply_on(c, down, out_dev, (const float *)c->g.p, 1, nullptr, st);
}

extern "C" int moty_cuda_ffn(MotyCudaMat *gate, MotyCudaMat *up, MotyCudaMat *down, int act,
                             float *out, const float *x, int S) {
    if (!gate || !up || !down || !out || !x) return moty_set_error(MOTY_CUDA_EARG, "ffn: null argument");
    DevCtx *c = moty_ctx(gate->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", gate->device);
    MOTY_USE_DEVICE(gate->device);
    if (S <= 0) return 0;
    size_t xb = (size_t)S * gate->I * 4;
    CKR(moty_grow(c, &c->dx, xb));
    CKR(moty_grow(c, &c->dy, xb));
    CK(cudaMemcpyAsync(c->dx.p, x, xb, cudaMemcpyHostToDevice, c->stream));
    CKR(ffn_on(c, gate, up, down, act, (float *)c->dy.p, (const float *)c->dx.p, S, c->stream));
    CK(cudaMemcpyAsync(out, c->dy.p, xb, cudaMemcpyDeviceToHost, c->stream));
    int kerr = 0;
    if (S == 1) CK(cudaMemcpyAsync(&kerr, c->err_dev + 1, 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    if (kerr) {
        cudaMemsetAsync(c->err_dev + 1, 0, 4, c->stream);
        cudaMemsetAsync(reinterpret_cast<unsigned *>(c->ctr) + 4, 0, 8, c->stream);
        return moty_set_error(MOTY_CUDA_EKERNEL, "fused FFN decode gave up on its grid barrier (result incomplete)");
    }
    return 0;
}

// ---------------------------------------------------------------------------
// MoE layer
// ---------------------------------------------------------------------------
struct MotyCudaMoe {
    int E, K, I, D, efmt, e_lo, e_hi, device;
    void *g, *u, *d;             // code slabs [e_hi - e_lo][...]
    void *gs, *us, *ds;          // scale slabs
    size_t gcb, gsb, dcb, dsb;   // bytes per expert: gate/up codes, gate/up scales, down codes, down scales
    MotyCudaMat *router;
    int sigmoid;                 // 1: LFM2's gate (sigmoid + expert bias) instead of softmax
    float *bias;                 // [E] on the device, or null
    // plan buffers (device), sized for capS tokens
    int capS;
    int *idx, *pair_tok, *pos_of, *ord, *counters;
    float *w, *ones;
    uint8_t *form;
    void *t_gate, *t_up, *t_down;
    float *logits;
};

extern "C" int moty_cuda_moe_create(MotyCudaMoe **out, int E, int K, int I, int D, int efmt,
                                    int e_lo, int e_hi, int device) {
    if (!out) return moty_set_error(MOTY_CUDA_EARG, "moe_create: null");
    DevCtx *c = moty_ctx(device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", device);
    if (E <= 0 || E > 4096 || K <= 0 || K > 64 || K > E || I <= 0 || D <= 0 || e_lo < 0 || e_hi > E || e_lo >= e_hi)
        return moty_set_error(MOTY_CUDA_EARG, "moe_create: E=%d K=%d I=%d D=%d experts [%d,%d)", E, K, I, D, e_lo, e_hi);
    if (efmt != MOTY_WF_I8 && efmt != MOTY_WF_Q4R4) return moty_set_error(MOTY_CUDA_EARG, "moe_create: expert format %d", efmt);
    if (efmt == MOTY_WF_I8 && (I % 16 || D % 16)) return moty_set_error(MOTY_CUDA_EARG, "moe_create: int8 experts need I, D %% 16 == 0");
    if (efmt == MOTY_WF_Q4R4 && (I % 32 || D % 32)) return moty_set_error(MOTY_CUDA_EARG, "moe_create: Q4R4 experts need I, D %% 32 == 0");
    if (I > MOTY_QROW_MAX || D > MOTY_QROW_MAX) return moty_set_error(MOTY_CUDA_ELIMIT, "moe_create: width above %d", MOTY_QROW_MAX);
    MOTY_USE_DEVICE(device);
    MotyCudaMoe *m = new (std::nothrow) MotyCudaMoe();
    if (!m) return moty_set_error(MOTY_CUDA_ENOMEM, "moe_create: host allocation");
    memset(m, 0, sizeof *m);
    m->E = E; m->K = K; m->I = I; m->D = D; m->efmt = efmt; m->e_lo = e_lo; m->e_hi = e_hi; m->device = device;
    CKR(mat_sizes(efmt, I, D, &m->gcb, &m->gsb));
    CKR(mat_sizes(efmt, D, I, &m->dcb, &m->dsb));
    size_t n = (size_t)(e_hi - e_lo);
    cudaError_t e = cudaMalloc(&m->g, n * m->gcb + 256);
    if (e == cudaSuccess) e = cudaMalloc(&m->u, n * m->gcb + 256);
    if (e == cudaSuccess) e = cudaMalloc(&m->d, n * m->dcb + 256);
    if (e == cudaSuccess) e = cudaMalloc(&m->gs, n * m->gsb + 256);
    if (e == cudaSuccess) e = cudaMalloc(&m->us, n * m->gsb + 256);
    if (e == cudaSuccess) e = cudaMalloc(&m->ds, n * m->dsb + 256);
    if (e != cudaSuccess) { moty_cuda_moe_free(m); return moty_set_error(MOTY_CUDA_ENOMEM, "moe_create: %s", cudaGetErrorString(e)); }
    *out = m;
    return 0;
}

static void moe_free_plan(MotyCudaMoe *m) {
    void *ps[] = {m->idx, m->pair_tok, m->pos_of, m->ord, m->counters, m->w, m->ones, m->form, m->t_gate, m->t_up, m->t_down, m->logits};
    for (void *p : ps) if (p) cudaFree(p);
    m->idx = m->pair_tok = m->pos_of = m->ord = m->counters = nullptr; m->w = nullptr; m->ones = nullptr; m->form = nullptr;
    m->t_gate = m->t_up = m->t_down = nullptr; m->logits = nullptr; m->capS = 0;
}

extern "C" int moty_cuda_moe_free(MotyCudaMoe *m) {
    if (!m) return 0;
    DevCtx *c = moty_ctx(m->device);
    if (c) { cudaSetDevice(m->device); cudaStreamSynchronize(c->stream); }
    void *ps[] = {m->g, m->u, m->d, m->gs, m->us, m->ds, m->bias};
    for (void *p : ps) if (p) cudaFree(p);
    moe_free_plan(m);
    delete m;
    return 0;
}

extern "C" int moty_cuda_moe_upload_expert(MotyCudaMoe *m, int eid, const void *g, const void *gs,
                                           const void *u, const void *us, const void *d, const void *ds) {
    if (!m || !g || !gs || !u || !us || !d || !ds) return moty_set_error(MOTY_CUDA_EARG, "moe_upload_expert: null argument");
    if (eid < m->e_lo || eid >= m->e_hi) return moty_set_error(MOTY_CUDA_EARG, "moe_upload_expert: expert %d outside [%d,%d)", eid, m->e_lo, m->e_hi);
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    size_t le = (size_t)(eid - m->e_lo);
    CK(cudaMemcpyAsync((char *)m->g + le * m->gcb, g, m->gcb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->u + le * m->gcb, u, m->gcb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->d + le * m->dcb, d, m->dcb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->gs + le * m->gsb, gs, m->gsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->us + le * m->gsb, us, m->gsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->ds + le * m->dsb, ds, m->dsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

// LFM2's int4 experts (ebits <= 4; nn/moe.c:42,99-103,138,193-198): the nibble rows are expanded to the codes nibble - 8
// on the way in and live in the layer's int8 slabs, so every int8 path (decode, batches, expert-parallel routes, both
// gates) serves them with the reference's integer sums.  Twice the bytes of a packed layout in HBM.
extern "C" int moty_cuda_moe_upload_expert_i4(MotyCudaMoe *m, int eid, const void *g4, const float *gs,
                                              const void *u4, const float *us, const void *d4, const float *ds) {
    if (!m || !g4 || !gs || !u4 || !us || !d4 || !ds) return moty_set_error(MOTY_CUDA_EARG, "moe_upload_expert_i4: null argument");
    if (m->efmt != MOTY_WF_I8) return moty_set_error(MOTY_CUDA_EARG, "moe_upload_expert_i4: the layer must be created with MOTY_WF_I8 experts");
    if (eid < m->e_lo || eid >= m->e_hi) return moty_set_error(MOTY_CUDA_EARG, "moe_upload_expert_i4: expert %d outside [%d,%d)", eid, m->e_lo, m->e_hi);
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    const size_t le = (size_t)(eid - m->e_lo);
    const size_t gb4 = (size_t)m->I * ((m->D + 1) / 2), db4 = (size_t)m->D * ((m->I + 1) / 2);
    CKR(moty_grow(c, &c->daux, 2 * gb4 + db4));
    uint8_t *s4 = (uint8_t *)c->daux.p;
    CK(cudaMemcpyAsync(s4, g4, gb4, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(s4 + gb4, u4, gb4, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(s4 + 2 * gb4, d4, db4, cudaMemcpyHostToDevice, c->stream));
    CKR(launch_i4_rows_to_i8(s4, (int8_t *)m->g + le * m->gcb, m->I, m->D, c->stream));
    CKR(launch_i4_rows_to_i8(s4 + gb4, (int8_t *)m->u + le * m->gcb, m->I, m->D, c->stream));
    CKR(launch_i4_rows_to_i8(s4 + 2 * gb4, (int8_t *)m->d + le * m->dcb, m->D, m->I, c->stream));
    CK(cudaMemcpyAsync((char *)m->gs + le * m->gsb, gs, m->gsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->us + le * m->gsb, us, m->gsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync((char *)m->ds + le * m->dsb, ds, m->dsb, cudaMemcpyHostToDevice, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    return 0;
}

extern "C" int moty_cuda_moe_set_router(MotyCudaMoe *m, MotyCudaMat *router) {
    if (!m) return moty_set_error(MOTY_CUDA_EARG, "moe_set_router: null");
    if (router && (router->O != m->E || router->I != m->D || router->device != m->device))
        return moty_set_error(MOTY_CUDA_EARG, "moe_set_router: router %dx%d on device %d", router->O, router->I, router->device);
    m->router = router;
    return 0;
}

extern "C" int moty_cuda_moe_set_sigmoid_gate(MotyCudaMoe *m, int on, const float *expert_bias) {
    if (!m) return moty_set_error(MOTY_CUDA_EARG, "moe_set_sigmoid_gate: null");
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    CK(cudaStreamSynchronize(c->stream));
    if (m->bias) { CK(cudaFree(m->bias)); m->bias = nullptr; }
    m->sigmoid = on != 0;
    if (on && expert_bias) {
        CK(cudaMalloc(&m->bias, (size_t)m->E * 4));
        CK(cudaMemcpy(m->bias, expert_bias, (size_t)m->E * 4, cudaMemcpyHostToDevice));
    }
    return 0;
}

static int moe_ensure_plan(MotyCudaMoe *m, int S) {
    if (S <= m->capS) return 0;
    DevCtx *c = moty_ctx(m->device);
    CK(cudaStreamSynchronize(c->stream));
    moe_free_plan(m);
    int cap = S + S / 4 + 8;
    size_t SK = (size_t)cap * m->K;
    size_t ntile = SK + (size_t)(m->e_hi - m->e_lo);      // loose bound: one row per tile
    size_t tsz = m->efmt == MOTY_WF_I8 ? sizeof(Q8Tile) : sizeof(Q4Tile);
    CK(cudaMalloc(&m->idx, SK * 4)); CK(cudaMalloc(&m->pair_tok, SK * 4)); CK(cudaMalloc(&m->pos_of, SK * 4));
    CK(cudaMalloc(&m->ord, SK * 4)); CK(cudaMalloc(&m->counters, 64)); CK(cudaMalloc(&m->w, SK * 4));
    CK(cudaMalloc(&m->form, SK + 16));
    CK(cudaMalloc(&m->ones, SK * 4));
    {
        float *tmp = (float *)malloc(SK * 4);
        if (!tmp) return moty_set_error(MOTY_CUDA_ENOMEM, "moe plan: host allocation");
        for (size_t i = 0; i < SK; i++) tmp[i] = 1.f;
        cudaError_t e = cudaMemcpy(m->ones, tmp, SK * 4, cudaMemcpyHostToDevice);
        free(tmp);
        CK(e);
    }
    CK(cudaMalloc(&m->t_gate, ntile * tsz)); CK(cudaMalloc(&m->t_up, ntile * tsz)); CK(cudaMalloc(&m->t_down, ntile * tsz));
    CK(cudaMalloc(&m->logits, (size_t)cap * m->E * 4));
    m->capS = cap;
    return 0;
}

// 0: generic tile path; 1: best decode path (one fused launch where supported); 2: the split
// decode path (router, gate/up and down as separate launches)

extern "C" int moty_cuda_set_moe_batch_path(int tensor_core) {
    int prev = g_moe_tc;
    g_moe_tc = tensor_core != 0;
    return prev;
}

extern "C" int moty_cuda_set_moe_fast_path(int on) {
    int prev = g_moe_fast;
    g_moe_fast = on < 0 ? 0 : (on > 3 ? 1 : on);
    return prev;
}

// eid_given == null: route the S tokens (softmax + top-K of the logits) and combine their K
// expert outputs in `order`.  eid_given != null: S rows with ONE given expert each (the rows an
// expert-parallel peer sent here); out[i] is that expert's output for row i, zero when the
// expert is not resident on this GPU.
static int moe_apply_on(DevCtx *c, MotyCudaMoe *m, float *out, const float *x, int S, const float *logits,
                        int order, int norm_topk, int *idx_out, float *w_out, const int *eid_given, cudaStream_t st,
                        float *rows = nullptr, float *const *rows_peer = nullptr, int npeer = 0) {
    const int E = m->E, K = eid_given ? 1 : m->K, I = m->I, D = m->D;
    const bool q8 = m->efmt == MOTY_WF_I8;
    // rows per tile of the grouped products: 8 for the int8 tile kernel; 8, 16 or 32 for the Q4R4 MMA kernel
    // (more when experts see more rows each)
    int T = 8;
    const long long per = (long long)S * K / E;                // routed rows an expert sees on average
    T = per >= 24 ? 32 : (per >= 12 ? 16 : 8);
    // batches whose experts see enough rows each take the tensor-core path (moe_tc.cu); its tiles are 16..128 rows
    const bool tc = q8 && g_moe_tc && per >= 8 && moe_tc_supported(I, D) && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (tc) T = moe_tc_tile_rows(per);
    CKR(moe_ensure_plan(m, eid_given ? (S + m->K - 1) / m->K : S));
    const int *idxp = m->idx; const float *wp = m->w;
    if (eid_given) {
        idxp = eid_given; wp = m->ones;
    } else {
        if (!logits) {
            if (!m->router) return moty_set_error(MOTY_CUDA_EARG, "moe: neither logits nor a router matrix");
            CKR(mat_apply_on(c, m->router, m->logits, x, S, nullptr, st));
            logits = m->logits;
        }
        // decode, int8 experts, softmax gate, nothing to exchange: two chained launches -- route + gate/up + SiLU, then
        // down + ordered sum.  (Measured against the one-launch cooperative kernel below, which cannot be chained to its
        // neighbours by programmatic dependent launch: see the dense FFN above.)
        if (S == 1 && q8 && order == 0 && g_moe_fast == 1 && !m->sigmoid && !rows && !npeer && E <= 2048 &&
            moe_decode_q8_supported(K, I, D) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            CKR(moty_grow(c, &c->g, (size_t)K * I * 4));
            CKR(launch_moe_decode_q8(m->idx, m->w, (const int8_t *)m->g, (const int8_t *)m->u, (const int8_t *)m->d,
                                     (const float *)m->gs, (const float *)m->us, (const float *)m->ds,
                                     m->gcb, m->gsb / 4, m->dcb, m->dsb / 4, x, (float *)c->g.p, out,
                                     K, I, D, m->e_lo, m->e_hi, c->sms, st, logits, E, norm_topk));
            if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            if (w_out) CK(cudaMemcpyAsync(w_out, m->w, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            return 0;
        }
        // the same in one cooperative launch (router, gate/up, bounded grid barrier, down): the expert-parallel decode
        // routes (row table, peer tables) live in this kernel, and set_moe_fast_path(3) sends every decode token here
        // (the one-launch kernels carry the softmax gate; the sigmoid gate takes the router launch + the two streaming launches)
        if (S == 1 && q8 && order == 0 && moe_fast_one() && !m->sigmoid && moe_decode_fused_q8_supported(E, K, I, D) &&
            (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            CKR(moty_grow(c, &c->g, (size_t)K * I * 4));
            CKR(launch_moe_decode_fused_q8(logits, E, norm_topk, m->idx, m->w, (const int8_t *)m->g, (const int8_t *)m->u,
                                           (const int8_t *)m->d, (const float *)m->gs, (const float *)m->us,
                                           (const float *)m->ds, m->gcb, m->gsb / 4, m->dcb, m->dsb / 4, x,
                                           (float *)c->g.p, out, rows, K, I, D, m->e_lo, m->e_hi,
                                           reinterpret_cast<unsigned *>(c->ctr) + 4, c->err_dev + 1, c->sms, st, rows_peer, npeer));
            if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            if (w_out) CK(cudaMemcpyAsync(w_out, m->w, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            return 0;
        }
        if (S == 1 && !q8 && order == 0 && moe_fast_one() && !m->sigmoid && moe_decode_fused_q4_supported(E, K, I, D) &&
            (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            CKR(moty_grow(c, &c->hq, (size_t)K * I + 16));
            CKR(moty_grow(c, &c->hxs, (size_t)K * (I / 32) * 4));
            CKR(moty_grow(c, &c->hxsum, (size_t)K * (I / 32) * 4));
            CKR(launch_moe_decode_fused_q4(logits, E, norm_topk, m->idx, m->w, (const uint8_t *)m->g, (const uint8_t *)m->u,
                                           (const uint8_t *)m->d, (const uint16_t *)m->gs, (const uint16_t *)m->us,
                                           (const uint16_t *)m->ds, m->gcb, m->gsb / 2, m->dcb, m->dsb / 2, x,
                                           (int8_t *)c->hq.p, (float *)c->hxs.p, (int *)c->hxsum.p, out, rows, K, I, D,
                                           m->e_lo, m->e_hi, reinterpret_cast<unsigned *>(c->ctr) + 4, c->err_dev + 1,
                                           c->sms, st, rows_peer, npeer,
                                           // nothing to exchange: the same kernel as two chained launches (see the int8 route above;
                                           // with the peer exchange behind it the one launch measured 1 us better: 29.7 / 30.9 us)
                                           (g_moe_fast == 1 && !rows && !npeer) ? 1 : 0));
            if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            if (w_out) CK(cudaMemcpyAsync(w_out, m->w, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
            return 0;
        }
        if (rows || npeer) return moty_set_error(MOTY_CUDA_ELIMIT, "moe_d1_rows: this layer (sigmoid gate, or shape E=%d K=%d I=%d D=%d) has no one-launch decode kernel", E, K, I, D);
        CKR(launch_route(logits, S, E, K, m->idx, m->w, nullptr, m->sigmoid ? 2 : 1, norm_topk, st, m->bias));
    }
    // decode fast path: one token, int8 experts, selection-order combine -> two streaming kernels
    if (S == 1 && q8 && !eid_given && order == 0 && g_moe_fast && moe_decode_q8_supported(K, I, D) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        CKR(moty_grow(c, &c->g, (size_t)K * I * 4));
        CKR(launch_moe_decode_q8(m->idx, m->w, (const int8_t *)m->g, (const int8_t *)m->u, (const int8_t *)m->d,
                                 (const float *)m->gs, (const float *)m->us, (const float *)m->ds,
                                 m->gcb, m->gsb / 4, m->dcb, m->dsb / 4, x, (float *)c->g.p, out,
                                 K, I, D, m->e_lo, m->e_hi, c->sms, st));
        if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
        if (w_out) CK(cudaMemcpyAsync(w_out, m->w, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
        return 0;
    }
    if (S == 1 && !q8 && !eid_given && order == 0 && g_moe_fast && moe_decode_q4_supported(K, I, D) &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        CKR(moty_grow(c, &c->g, (size_t)K * I * 4));
        CKR(launch_moe_decode_q4(m->idx, m->w, (const uint8_t *)m->g, (const uint8_t *)m->u, (const uint8_t *)m->d,
                                 (const uint16_t *)m->gs, (const uint16_t *)m->us, (const uint16_t *)m->ds,
                                 m->gcb, m->gsb / 2, m->dcb, m->dsb / 2, x, (float *)c->g.p, out,
                                 K, I, D, m->e_lo, m->e_hi, c->sms, st));
        if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
        if (w_out) CK(cudaMemcpyAsync(w_out, m->w, (size_t)K * 4, cudaMemcpyDeviceToDevice, st));
        return 0;
    }
    size_t P = (size_t)S * K;                                 // upper bound on local (token, expert) pairs
    int ntiles_max = (int)((P + T - 1) / T) + (m->e_hi - m->e_lo);
    if ((size_t)ntiles_max > P + (size_t)(m->e_hi - m->e_lo)) ntiles_max = (int)(P + (size_t)(m->e_hi - m->e_lo));
    if (ntiles_max > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "moe: %d tiles in one call; split the batch", ntiles_max);
    MoePlanArgs pa; memset(&pa, 0, sizeof pa);
    pa.idx = idxp; pa.S = S; pa.K = K; pa.E = E; pa.e_lo = m->e_lo; pa.e_hi = m->e_hi; pa.T = T; pa.order = order; pa.q8 = q8;
    if (q8) {
        pa.g8 = (const int8_t *)m->g; pa.u8 = (const int8_t *)m->u; pa.d8 = (const int8_t *)m->d;
        pa.gs = (const float *)m->gs; pa.us = (const float *)m->us; pa.ds = (const float *)m->ds;
        pa.gstride = m->gcb; pa.gsstride = m->gsb / 4; pa.dstride = m->dcb; pa.dsstride = m->dsb / 4;
        pa.t8_gate = (Q8Tile *)m->t_gate; pa.t8_up = (Q8Tile *)m->t_up; pa.t8_down = (Q8Tile *)m->t_down;
    } else {
        pa.g4 = (const uint8_t *)m->g; pa.u4 = (const uint8_t *)m->u; pa.d4 = (const uint8_t *)m->d;
        pa.gs16 = (const uint16_t *)m->gs; pa.us16 = (const uint16_t *)m->us; pa.ds16 = (const uint16_t *)m->ds;
        pa.gstride = m->gcb; pa.gsstride = m->gsb / 2; pa.dstride = m->dcb; pa.dsstride = m->dsb / 2;
        pa.t4_gate = (Q4Tile *)m->t_gate; pa.t4_up = (Q4Tile *)m->t_up; pa.t4_down = (Q4Tile *)m->t_down;
        pa.form = m->form;
    }
    pa.pair_tok = m->pair_tok; pa.pos_of = m->pos_of; pa.ord = m->ord;
    pa.ntiles = m->counters; pa.npairs = m->counters + 1;
    CKR(launch_moe_plan(pa, st));

    // activations of the two halves: [P][I] each, then the down outputs [P][D]
    CKR(moty_grow(c, &c->g, P * I * 4));
    CKR(moty_grow(c, &c->u, P * I * 4));
    CKR(moty_grow(c, &c->h, P * D * 4));
    if (tc) {
        // gather folded into the row quantizer, gate+up+SiLU in one tensor-core pass, row quantizer, down pass
        const int El = m->e_hi - m->e_lo;
        CKR(moty_grow(c, &c->xi, P * D + 1024));
        CKR(moty_grow(c, &c->sx, P * 4));
        CKR(moty_grow(c, &c->hq, P * I + 1024));
        CKR(moty_grow(c, &c->hs, P * 4));
        CKR(launch_qrow_i8_scatter(x, m->pos_of, S, K, (int8_t *)c->xi.p, (float *)c->sx.p, D, st));
        CKR(launch_moe_tc_gateup((const Q8Tile *)m->t_gate, (const Q8Tile *)m->t_up, m->counters, T, (const int8_t *)m->g,
                                 (const int8_t *)m->u, El, (const int8_t *)c->xi.p, (const float *)c->sx.p, (int)P,
                                 (float *)c->g.p, I, D, c->err_dev, c->sms, st));
        CKR(launch_qrow_i8_counted((const float *)c->g.p, (int8_t *)c->hq.p, (float *)c->hs.p, (int)P, I, m->counters + 1, st));
        CKR(launch_moe_tc_down((const Q8Tile *)m->t_down, m->counters, T, (const int8_t *)m->d, El, (const int8_t *)c->hq.p,
                               (const float *)c->hs.p, (int)P, (float *)c->h.p, I, D, c->err_dev, c->sms, st));
    } else if (q8) {
        CK(cudaMemsetAsync(c->g.p, 0, P * I * 4, st));
        CK(cudaMemsetAsync(c->u.p, 0, P * I * 4, st));
        CKR(moty_grow(c, &c->xi, (size_t)S * D + 16));
        CKR(moty_grow(c, &c->sx, (size_t)S * 4));
        CKR(moty_grow(c, &c->hq, P * I + 16));
        CKR(moty_grow(c, &c->hs, P * 4));
        CKR(launch_qrow_i8(x, (int8_t *)c->xi.p, (float *)c->sx.p, S, D, st));
        CKR(launch_q8_mma_grouped((const Q8Tile *)m->t_gate, m->counters, ntiles_max, T, (const int8_t *)c->xi.p,
                                  (const float *)c->sx.p, m->pair_tok, (float *)c->g.p, I, D, I, st));
        CKR(launch_q8_mma_grouped((const Q8Tile *)m->t_up, m->counters, ntiles_max, T, (const int8_t *)c->xi.p,
                                  (const float *)c->sx.p, m->pair_tok, (float *)c->u.p, I, D, I, st));
        CKR(launch_act_mul((float *)c->g.p, (const float *)c->u.p, (int64_t)P * I, MOTY_ACT_SILU, st));
        CKR(launch_qrow_i8((const float *)c->g.p, (int8_t *)c->hq.p, (float *)c->hs.p, (int)P, I, st));
        CKR(launch_q8_mma_grouped((const Q8Tile *)m->t_down, m->counters, ntiles_max, T, (const int8_t *)c->hq.p,
                                  (const float *)c->hs.p, nullptr, (float *)c->h.p, D, I, D, st));
    } else {
        // rows the plan leaves unused (non-local experts) must not feed NaNs to the quantizers
        CK(cudaMemsetAsync(c->g.p, 0, P * I * 4, st));
        CK(cudaMemsetAsync(c->u.p, 0, P * I * 4, st));
        int nbD = D / 32, nbI = I / 32;
        CKR(moty_grow(c, &c->xi, (size_t)S * D + 16));
        CKR(moty_grow(c, &c->xs, (size_t)S * nbD * 4));
        CKR(moty_grow(c, &c->xsum, (size_t)S * nbD * 4));
        CKR(moty_grow(c, &c->hq, P * I + 16));
        CKR(moty_grow(c, &c->hxs, P * nbI * 4));
        CKR(moty_grow(c, &c->hxsum, P * nbI * 4));
        CKR(launch_quant_g32(x, S, D, (int8_t *)c->xi.p, (float *)c->xs.p, (int32_t *)c->xsum.p, st));
        const size_t P8 = (P + 7) / 8 * 8;
        CKR(moty_grow(c, &c->rec, P8 * (size_t)(nbD > nbI ? nbD : nbI) * 16));
        CKR(launch_q4r4_mma_grouped((const Q4Tile *)m->t_gate, m->counters, ntiles_max, T, m->counters + 1,
                                    (const int8_t *)c->xi.p, (const float *)c->xs.p, (const int32_t *)c->xsum.p,
                                    m->pair_tok, m->form, (int4 *)c->rec.p, 1, (float *)c->g.p, I, (int)P, D, I, st, g_q4r4_relaxed, c->sms));
        CKR(launch_q4r4_mma_grouped((const Q4Tile *)m->t_up, m->counters, ntiles_max, T, m->counters + 1,
                                    (const int8_t *)c->xi.p, (const float *)c->xs.p, (const int32_t *)c->xsum.p,
                                    m->pair_tok, m->form, (int4 *)c->rec.p, 0, (float *)c->u.p, I, (int)P, D, I, st, g_q4r4_relaxed, c->sms));
        CKR(launch_act_mul((float *)c->g.p, (const float *)c->u.p, (int64_t)P * I, MOTY_ACT_SILU, st));
        CKR(launch_quant_g32((const float *)c->g.p, (int)P, I, (int8_t *)c->hq.p, (float *)c->hxs.p, (int32_t *)c->hxsum.p, st));
        CKR(launch_q4r4_mma_grouped((const Q4Tile *)m->t_down, m->counters, ntiles_max, T, m->counters + 1,
                                    (const int8_t *)c->hq.p, (const float *)c->hxs.p, (const int32_t *)c->hxsum.p,
                                    nullptr, m->form, (int4 *)c->rec.p, 1, (float *)c->h.p, D, (int)P, I, D, st, g_q4r4_relaxed, c->sms));
    }
    CKR(launch_moe_combine(out, (const float *)c->h.p, wp, m->pos_of, m->ord, S, K, D, st));
    if (idx_out) CK(cudaMemcpyAsync(idx_out, m->idx, P * 4, cudaMemcpyDeviceToDevice, st));
    if (w_out) CK(cudaMemcpyAsync(w_out, m->w, P * 4, cudaMemcpyDeviceToDevice, st));
    return 0;
}

extern "C" int moty_cuda_moe_apply_dev(MotyCudaMoe *m, float *out_dev, const float *x_dev, int S,
                                       const float *logits_dev, int order, int norm_topk,
                                       int *idx_dev, float *w_dev, void *stream) {
    if (!m || !out_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "moe_apply_dev: null argument");
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    if (S <= 0) return 0;
    return moe_apply_on(c, m, out_dev, x_dev, S, logits_dev, order, norm_topk, idx_dev, w_dev, nullptr, pick_stream(c, stream));
}

static int moe_host(MotyCudaMoe *m, float *out, const float *x, int S, const float *logits, int order, int norm) {
    if (!m || !out || !x) return moty_set_error(MOTY_CUDA_EARG, "moe: null argument");
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    if (S <= 0) return 0;
    size_t xb = (size_t)S * m->D * 4, lb = (size_t)S * m->E * 4;
    CKR(moty_grow(c, &c->dx, xb));
    CKR(moty_grow(c, &c->dy, xb));
    CK(cudaMemcpyAsync(c->dx.p, x, xb, cudaMemcpyHostToDevice, c->stream));
    const float *dl = nullptr;
    if (logits) {
        CKR(moty_grow(c, &c->dlogits, lb));
        CK(cudaMemcpyAsync(c->dlogits.p, logits, lb, cudaMemcpyHostToDevice, c->stream));
        dl = (const float *)c->dlogits.p;
    }
    CKR(moe_apply_on(c, m, (float *)c->dy.p, (const float *)c->dx.p, S, dl, order, norm, nullptr, nullptr, nullptr, c->stream));
    CK(cudaMemcpyAsync(out, c->dy.p, xb, cudaMemcpyDeviceToHost, c->stream));
    int kerr = 0;
    CK(cudaMemcpyAsync(&kerr, c->err_dev + 1, 4, cudaMemcpyDeviceToHost, c->stream));
    CK(cudaStreamSynchronize(c->stream));
    if (kerr) {
        // the grid barrier of the fused decode kernel expired: its counters are no longer consistent
        cudaMemsetAsync(c->err_dev + 1, 0, 4, c->stream);
        cudaMemsetAsync(c->ctr + 4, 0, 8, c->stream);
        return moty_set_error(MOTY_CUDA_EKERNEL, "fused MoE decode gave up on its grid barrier (result incomplete)");
    }
    return 0;
}

extern "C" int moty_cuda_moe_d1(MotyCudaMoe *m, float *out, const float *x, const float *logits) {
    return moe_host(m, out, x, 1, logits, 0, 1);
}

extern "C" int moty_cuda_moe_batch(MotyCudaMoe *m, float *out, const float *x, int S, const float *logits) {
    return moe_host(m, out, x, S, logits, 1, 1);
}

extern "C" int moty_cuda_olmoe_moe(MotyCudaMoe *m, float *out, const float *x, int S, const float *logits, int norm_topk) {
    return moe_host(m, out, x, S, logits, 0, norm_topk);
}

// ---------------------------------------------------------------------------
// expert-parallel building blocks (device pointers)
// ---------------------------------------------------------------------------
extern "C" int moty_cuda_moe_d1_rows_dev(MotyCudaMoe *m, float *rows_dev, float *out_dev, const float *x_dev,
                                         const float *logits_dev, int norm_topk, int *idx_dev, float *w_dev, void *stream) {
    if (!m || !rows_dev || !out_dev || !x_dev) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_rows_dev: null argument");
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    if (!moe_fast_one()) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_rows_dev needs the one-launch decode path (set_moe_fast_path(1))");
    if (reinterpret_cast<uintptr_t>(x_dev) & 15) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_rows_dev: x_dev must be 16-byte aligned");
    return moe_apply_on(c, m, out_dev, x_dev, 1, logits_dev, 0, norm_topk, idx_dev, w_dev, nullptr, pick_stream(c, stream), rows_dev);
}

extern "C" int moty_cuda_moe_d1_peer_dev(MotyCudaMoe *m, float *out_dev, const float *x_dev, const float *logits_dev, int norm_topk,
                                         void *const *tables, void *const *flags, int world, int rank, unsigned epoch,
                                         void *stream) {
    if (!m || !out_dev || !x_dev || !tables || !flags) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_peer_dev: null argument");
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_peer_dev: rank %d of %d (1..8 ranks)", rank, world);
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    if (!moe_fast_one()) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_peer_dev needs the one-launch decode path (set_moe_fast_path(1))");
    if (reinterpret_cast<uintptr_t>(x_dev) & 15) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_peer_dev: x_dev must be 16-byte aligned");
    cudaStream_t st = pick_stream(c, stream);
    float *tb[8]; unsigned *fl[8];
    const size_t half = (size_t)m->K * m->D;                       // two tables per rank, used alternately
    for (int r = 0; r < world; r++) {
        if (!tables[r] || !flags[r]) return moty_set_error(MOTY_CUDA_EARG, "moe_d1_peer_dev: null table or flag pointer for rank %d", r);
        tb[r] = (float *)tables[r] + (epoch & 1u) * half;
        fl[r] = (unsigned *)flags[r];
    }
    CKR(moe_apply_on(c, m, out_dev, x_dev, 1, logits_dev, 0, norm_topk, nullptr, nullptr, nullptr, st, nullptr, tb, world));
    return launch_moe_peer_combine(out_dev, tb[rank], m->w, m->idx, m->K, m->D, fl, fl[rank], world, rank, epoch, c->err_dev + 1, st);
}

extern "C" int moty_cuda_moe_experts_dev(MotyCudaMoe *m, float *h_dev, const float *x_rows_dev, const int *eid_dev,
                                         int P, void *stream) {
    if (!m || !h_dev || !x_rows_dev || !eid_dev) return moty_set_error(MOTY_CUDA_EARG, "moe_experts_dev: null argument");
    DevCtx *c = moty_ctx(m->device);
    if (!c) return moty_set_error(MOTY_CUDA_EINIT, "device %d not initialised", m->device);
    MOTY_USE_DEVICE(m->device);
    if (P <= 0) return 0;
    return moe_apply_on(c, m, h_dev, x_rows_dev, P, nullptr, 0, 0, nullptr, nullptr, eid_dev, pick_stream(c, stream));
}

extern "C" int moty_cuda_moe_combine_dev(float *out_dev, const float *h_dev, const float *w_dev, const int *idx_dev,
                                         int S, int K, int D, int order, void *stream) {
    if (!out_dev || !h_dev || !w_dev || !idx_dev) return moty_set_error(MOTY_CUDA_EARG, "moe_combine_dev: null argument");
    if (S <= 0) return 0;
    if (K < 1 || K > 64 || D < 1) return moty_set_error(MOTY_CUDA_EARG, "moe_combine_dev: K=%d D=%d", K, D);
    MOTY_CTX_OF(out_dev, c);
    return launch_moe_combine_sk(out_dev, h_dev, w_dev, idx_dev, S, K, D, order, pick_stream(c, stream));
}
