// gemv_q8.cu -- Q8_0 products for few activation rows (decode and small batches).
//
// HBM-bound integer work: every weight byte is read once with 128-bit
// L1-bypassing loads, the quantized activation rows sit in shared memory, the
// int8 x int8 products go through dp4a into int32 accumulators, and a
// multi-value butterfly reduces a warp's R x NS partial sums in R*NS-1 shuffles.
// Replaces moty_matmul_q_s / q8_idot_rows (nn/matmul.c:29-36, 51-66).
#include "kernels.cuh"

// Reduce N (power of two, <= 32) per-lane values across the warp.  On return the
// lane L holds in v[0] the warp-wide sum of value number (L >> (5 - log2 N)).
template <int N>
__device__ __forceinline__ void warp_reduce_multi(int (&v)[N], int lane) {
    int off = 16;
#pragma unroll
    for (int n = N; n > 1; n >>= 1, off >>= 1) {
#pragma unroll
        for (int i = 0; i < n / 2; i++) {
            bool up = (lane & off) != 0;
            int send = up ? v[i] : v[i + n / 2];
            int keep = up ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    for (; off > 0; off >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
}

template <int N> struct Log2 { static constexpr int v = 1 + Log2<N / 2>::v; };
template <> struct Log2<1> { static constexpr int v = 0; };

// One warp: R weight rows starting at o0 against NS staged activation rows.
template <int NS, int R>
__device__ __forceinline__ void q8_rows(const int8_t *__restrict__ W, const int4 *__restrict__ xsm,
                                        int I16, int O, int o0, int lane, int (&flat)[R * NS]) {
    const int4 *wp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        int o = o0 + r < O ? o0 + r : O - 1;                 // tail rows re-read the last row, never stored
        wp[r] = reinterpret_cast<const int4 *>(W + (size_t)o * I16 * 16);
    }
#pragma unroll
    for (int i = 0; i < R * NS; i++) flat[i] = 0;
#pragma unroll 2
    for (int k = lane; k < I16; k += 32) {
        int4 wv[R];
#pragma unroll
        for (int r = 0; r < R; r++) wv[r] = ldg_stream16(wp[r] + k);
#pragma unroll
        for (int s = 0; s < NS; s++) {
            int4 xv = xsm[s * I16 + k];
#pragma unroll
            for (int r = 0; r < R; r++) flat[r * NS + s] = dp4a4(wv[r], xv, flat[r * NS + s]);
        }
    }
    warp_reduce_multi<R * NS>(flat, lane);
}

template <int NS, int R>
__global__ void __launch_bounds__(256) q8_small_kernel(Q8Args a) {
    extern __shared__ int4 xsm[];                            // [NS][I/16]
    const int tile = blockIdx.y;
    const int8_t *W; const float *scale; int row0, nrows;
    if (a.tiles) {
        if (tile >= *a.ntiles_dev) return;
        Q8Tile t = a.tiles[tile];
        W = t.w; scale = t.scale; row0 = t.row0; nrows = t.nrows;
    } else {
        W = a.w; scale = a.scale; row0 = tile * NS;
        nrows = a.S - row0 < NS ? a.S - row0 : NS;
    }
    const int I16 = a.I / 16, O = a.O;
    for (int idx = threadIdx.x; idx < NS * I16; idx += 256) {
        int s = idx / I16, k = idx - s * I16;
        int4 v = make_int4(0, 0, 0, 0);
        if (s < nrows) {
            int xr = a.xmap ? a.xmap[row0 + s] : row0 + s;
            v = reinterpret_cast<const int4 *>(a.xi + (size_t)xr * a.I)[k];
        }
        xsm[idx] = v;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int SH = 5 - Log2<R * NS>::v;
    for (int rg = blockIdx.x * 8 + warp; rg * R < O; rg += gridDim.x * 8) {
        int flat[R * NS];
        q8_rows<NS, R>(W, xsm, I16, O, rg * R, lane, flat);
        if ((lane & ((1 << SH) - 1)) == 0) {
            int p = lane >> SH, r = p / NS, s = p % NS, o = rg * R + r;
            if (s < nrows && o < O) {
                int xr = a.xmap ? a.xmap[row0 + s] : row0 + s;
                int yr = a.ymap ? a.ymap[row0 + s] : row0 + s;
                // (scale[o] * sx[s]) * (float)dot, evaluated left to right (nn/matmul.c:34)
                float v = __fmul_rn(__fmul_rn(scale[o], a.sx[xr]), (float)flat[0]);
                a.y[(size_t)yr * a.ldy + o] = v;
                if (a.acc) a.acc[(size_t)yr * a.ldy + o] = flat[0];
            }
        }
    }
}

template <int NS, int R>
static int launch_small_t(const Q8Args &a, int ntile, int sms, cudaStream_t st) {
    size_t smem = (size_t)NS * a.I;
    int nrg = (a.O + R - 1) / R;
    int gx = (nrg + 7) / 8;
    // many tiles already fill the GPU: let each CTA walk more row groups so the
    // activation rows are staged less often
    if (ntile > 1) { int cap = (sms * 8 + ntile - 1) / ntile; if (cap < 1) cap = 1; if (gx > cap) gx = cap; }
    dim3 grid(gx, ntile);
    q8_small_kernel<NS, R><<<grid, 256, smem, st>>>(a);
    CK(cudaGetLastError());
    return 0;
}

template <int NS>
static int launch_small_ns(const Q8Args &a, int ntile, int sms, cudaStream_t st) {
    // R rows per warp: more rows = more loads in flight, fewer warps
    long long warps_r4 = (a.O + 3) / 4;
    if (NS <= 4 && warps_r4 * ntile >= (long long)sms * 16) return launch_small_t<NS, 4>(a, ntile, sms, st);
    if ((long long)(a.O + 1) / 2 * ntile >= (long long)sms * 8) return launch_small_t<NS, 2>(a, ntile, sms, st);
    return launch_small_t<NS, 1>(a, ntile, sms, st);
}

// opt in to large dynamic shared memory (8 rows x 16384 bytes); once per device
#define Q8_ATTR(NS, R) CK(cudaFuncSetAttribute(q8_small_kernel<NS, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024))
int gemv_q8_init_device() {
    Q8_ATTR(1, 1); Q8_ATTR(1, 2); Q8_ATTR(1, 4);
    Q8_ATTR(2, 1); Q8_ATTR(2, 2); Q8_ATTR(2, 4);
    Q8_ATTR(4, 1); Q8_ATTR(4, 2); Q8_ATTR(4, 4);
    Q8_ATTR(8, 1); Q8_ATTR(8, 2);
    return 0;
}

int launch_q8_small(const Q8Args &a, int sms, cudaStream_t st) {
    if (a.I % 16 != 0 || a.I > MOTY_QROW_MAX) return moty_set_error(MOTY_CUDA_EARG, "q8_small: I=%d", a.I);
    if (a.O <= 0 || a.S <= 0) return 0;
    if (a.tiles) return launch_small_ns<8>(a, a.ntiles_max, sms, st);
    if (a.S == 1) return launch_small_ns<1>(a, 1, sms, st);
    if (a.S == 2) return launch_small_ns<2>(a, 1, sms, st);
    if (a.S <= 4) return launch_small_ns<4>(a, 1, sms, st);
    return launch_small_ns<8>(a, (a.S + 7) / 8, sms, st);
}

// ---------------------------------------------------------------------------
// Any-length dots (test entries and widths that are not a multiple of 16):
// one warp per weight row, word loads where both pointers allow, bytes otherwise.
// moty_hw_dot_i8i8 (hw/hw_scalar.h:8-12), moty_hw_dot_i4i8 (:14-22).
// ---------------------------------------------------------------------------
__device__ __forceinline__ int dot_i8_any(const int8_t *__restrict__ w, const int8_t *__restrict__ x, int n, int lane) {
    int acc = 0;
    if (((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 3) == 0) {
        const int *w4 = reinterpret_cast<const int *>(w), *x4 = reinterpret_cast<const int *>(x);
        int n4 = n / 4;
        for (int i = lane; i < n4; i += 32) acc = __dp4a(w4[i], x4[i], acc);
        for (int i = n4 * 4 + lane; i < n; i += 32) acc += (int)w[i] * (int)x[i];
    } else {
        for (int i = lane; i < n; i += 32) acc += (int)w[i] * (int)x[i];
    }
    return warp_sum_i32(acc);
}

__device__ __forceinline__ int dot_i4_any(const uint8_t *__restrict__ w4, const int8_t *__restrict__ x, int n, int lane) {
    int acc = 0, rb = (n + 1) / 2;
    for (int b = lane; b < rb; b += 32) {
        int byte = w4[b];
        acc += ((byte & 15) - 8) * (int)x[2 * b];
        if (2 * b + 1 < n) acc += ((byte >> 4) - 8) * (int)x[2 * b + 1];
    }
    return warp_sum_i32(acc);
}

__global__ void __launch_bounds__(256) dot_i8i8_rows_kernel(const int8_t *w, const int8_t *x, int nrows, int n, int32_t *out) {
    int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= nrows) return;
    int d = dot_i8_any(w + (size_t)row * n, x, n, lane);
    if (lane == 0) out[row] = d;
}

__global__ void __launch_bounds__(256) dot_i4i8_rows_kernel(const uint8_t *w4, const int8_t *x, int nrows, int n, int32_t *out) {
    int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= nrows) return;
    int d = dot_i4_any(w4 + (size_t)row * ((n + 1) / 2), x, n, lane);
    if (lane == 0) out[row] = d;
}

int launch_dot_i8i8_rows(const int8_t *w, const int8_t *x, int nrows, int n, int32_t *out, cudaStream_t st) {
    if (nrows <= 0) return 0;
    dot_i8i8_rows_kernel<<<(nrows + 7) / 8, 256, 0, st>>>(w, x, nrows, n, out);
    CK(cudaGetLastError());
    return 0;
}

int launch_dot_i4i8_rows(const uint8_t *w4, const int8_t *x, int nrows, int n, int32_t *out, cudaStream_t st) {
    if (nrows <= 0) return 0;
    dot_i4i8_rows_kernel<<<(nrows + 7) / 8, 256, 0, st>>>(w4, x, nrows, n, out);
    CK(cudaGetLastError());
    return 0;
}

// generic Q8_0 rows for widths the vector kernel cannot take (I % 16 != 0)
__global__ void __launch_bounds__(256) q8_any_kernel(const int8_t *W, const float *scale, const int8_t *xi, const float *sx,
                                                     float *y, int32_t *acc, int S, int I, int O) {
    int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (o >= O) return;
    for (int s = 0; s < S; s++) {
        int d = dot_i8_any(W + (size_t)o * I, xi + (size_t)s * I, I, lane);
        if (lane == 0) {
            y[(size_t)s * O + o] = __fmul_rn(__fmul_rn(scale[o], sx[s]), (float)d);
            if (acc) acc[(size_t)s * O + o] = d;
        }
    }
}

int launch_q8_any(const int8_t *W, const float *scale, const int8_t *xi, const float *sx, float *y, int32_t *acc,
                  int S, int I, int O, cudaStream_t st) {
    if (O <= 0 || S <= 0) return 0;
    q8_any_kernel<<<(O + 7) / 8, 256, 0, st>>>(W, scale, xi, sx, y, acc, S, I, O);
    CK(cudaGetLastError());
    return 0;
}

