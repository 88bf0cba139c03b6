// q4r4.cu -- grouped-int4 "Q4R4" products (4-row blocks, groups of 32, f16 scales).
//
// Replaces moty_hw_q4r4_gemm_ref / _gemm4t_ref (hw/hw_q4r4.h:47-84) and the
// driver moty_matmul_q4r4_s (nn/matmul.c:405-433) for few activation rows.
//
// A warp owns one 4-row block.  Per step it reads 512 contiguous bytes of codes:
// lane = (group-in-step << 2) | row, 16 bytes each = the 32 nibbles of one
// (row, group).  Integer group sums are exact (dp4a on the split nibbles).
// The f32 accumulation is ONE sequential chain per (row, token) in ascending
// group order, exactly like the CPU loop: the running sum hops from the lane
// of group g to the lane of group g+1 by shuffle, one fused multiply-add per
// hop.  That costs 8 shuffles per 512 bytes and makes the result bit-identical
// to the reference instead of merely close.
#include "kernels.cuh"

template <int NS>
__global__ void __launch_bounds__(256) q4r4_small_kernel(Q4Args a) {
    extern __shared__ int4 sm4[];
    const int tile = blockIdx.y;
    const uint8_t *W; const uint16_t *Dsc; int row0, nrows;
    if (a.tiles) {
        if (tile >= *a.ntiles_dev) return;
        Q4Tile t = a.tiles[tile];
        W = t.w; Dsc = t.d; row0 = t.row0; nrows = t.nrows;
    } else {
        W = a.w; Dsc = a.d; row0 = tile * NS;
        nrows = a.S - row0 < NS ? a.S - row0 : NS;
    }
    const int I = a.I, nb = I / 32, I16 = I / 16, O = a.O;
    int8_t *xq_s = reinterpret_cast<int8_t *>(sm4);
    float *xs_s = reinterpret_cast<float *>(xq_s + (size_t)NS * I);
    int *xsum_s = reinterpret_cast<int *>(xs_s + (size_t)NS * nb);
    __shared__ int form_s[NS];
    for (int idx = threadIdx.x; idx < NS * I16; idx += 256) {
        int s = idx / I16, k = idx - s * I16;
        int4 v = make_int4(0, 0, 0, 0);
        if (s < nrows) {
            int xr = a.xmap ? a.xmap[row0 + s] : row0 + s;
            v = reinterpret_cast<const int4 *>(a.xq + (size_t)xr * I)[k];
        }
        sm4[idx] = v;
    }
    for (int idx = threadIdx.x; idx < NS * nb; idx += 256) {
        int s = idx / nb, g = idx - s * nb;
        float sc = 0.f; int sm = 0;
        if (s < nrows) {
            int xr = a.xmap ? a.xmap[row0 + s] : row0 + s;
            sc = a.xs[(size_t)xr * nb + g]; sm = a.xsum[(size_t)xr * nb + g];
        }
        xs_s[idx] = sc; xsum_s[idx] = sm;
    }
    if (threadIdx.x < NS) {
        int s = threadIdx.x, f = 0;
        if (s < nrows && a.form) f = a.form[row0 + s];
        form_s[s] = f;
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gl = lane >> 2, r = lane & 3;
    const int nblk = (O + 3) / 4, nit = (nb + 7) / 8;
    const int prev = (lane + 28) & 31;                       // the lane of the previous group, same row
    for (int ob = blockIdx.x * 8 + warp; ob < nblk; ob += gridDim.x * 8) {
        const uint8_t *wb = W + (size_t)ob * nb * 64;
        const uint16_t *db = Dsc + (size_t)ob * nb * 4;
        float acc[NS];
#pragma unroll
        for (int s = 0; s < NS; s++) acc[s] = 0.f;
        for (int it0 = 0; it0 < nit; it0 += 4) {
            int4 wv[4]; uint16_t dv[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {                      // up to 2 KB of codes in flight per warp
                int g = (it0 + u) * 8 + gl;
                wv[u] = make_int4(0, 0, 0, 0); dv[u] = 0;
                if (g < nb) {
                    wv[u] = ldg_stream16(wb + (size_t)(it0 + u) * 512 + lane * 16);
                    dv[u] = __ldg(db + (size_t)(it0 + u) * 32 + lane);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (it0 + u >= nit) break;
                const int g = (it0 + u) * 8 + gl;
                const bool valid = g < nb;
                const int gc = valid ? g : nb - 1;
                const float dd = f16bits_to_f32(dv[u]);
                int4 lo, hi;
                lo.x = wv[u].x & 0x0f0f0f0f; hi.x = (wv[u].x >> 4) & 0x0f0f0f0f;
                lo.y = wv[u].y & 0x0f0f0f0f; hi.y = (wv[u].y >> 4) & 0x0f0f0f0f;
                lo.z = wv[u].z & 0x0f0f0f0f; hi.z = (wv[u].z >> 4) & 0x0f0f0f0f;
                lo.w = wv[u].w & 0x0f0f0f0f; hi.w = (wv[u].w >> 4) & 0x0f0f0f0f;
                float fs[NS], c0[NS], c1[NS];
#pragma unroll
                for (int s = 0; s < NS; s++) {
                    const int4 *xg = reinterpret_cast<const int4 *>(xq_s + (size_t)s * I + gc * 32);
                    int4 x0 = xg[0], x1 = xg[1];
                    int sraw = dp4a4(lo, x0, 0);
                    sraw = dp4a4(hi, x1, sraw);
                    float xsc = xs_s[s * nb + gc];
                    int xsm = xsum_s[s * nb + gc];
                    if (form_s[s]) {
                        // 4-token tile (hw/hw_q4r4.h:78-81): raw sum scaled, offset folded in float
                        fs[s] = (float)sraw;
                        c0[s] = __fmul_rn(dd, xsc);
                        c1[s] = __fmul_rn(__fmul_rn(8.f, (float)xsm), xsc);
                    } else {
                        // token by token (hw/hw_q4r4.h:58-59): offset removed in the integers
                        fs[s] = (float)(sraw - 8 * xsm);
                        c0[s] = __fmul_rn(dd, xsc);
                        c1[s] = 0.f;
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; j++) {
#pragma unroll
                    for (int s = 0; s < NS; s++) {
                        float in = __shfl_sync(0xffffffffu, acc[s], prev);
                        if (gl == j) {
                            float t = in;
                            if (valid) {
                                t = fmaf(fs[s], c0[s], in);
                                if (form_s[s]) t = fmaf(-dd, c1[s], t);
                            }
                            acc[s] = t;
                        }
                    }
                }
            }
        }
        if (gl == 7) {
            int o = ob * 4 + r;
            if (o < O) {
#pragma unroll
                for (int s = 0; s < NS; s++)
                    if (s < nrows) {
                        int yr = a.ymap ? a.ymap[row0 + s] : row0 + s;
                        a.y[(size_t)yr * a.ldy + o] = acc[s];
                    }
            }
        }
    }
}

template <int NS>
static int launch_q4_t(const Q4Args &a, int ntile, int sms, cudaStream_t st) {
    int nb = a.I / 32;
    size_t smem = (size_t)NS * a.I + (size_t)NS * nb * 8;
    int nblk = (a.O + 3) / 4;
    int gx = (nblk + 7) / 8;
    if (ntile > 1) { int cap = (sms * 8 + ntile - 1) / ntile; if (cap < 1) cap = 1; if (gx > cap) gx = cap; }
    dim3 grid(gx, ntile);
    q4r4_small_kernel<NS><<<grid, 256, smem, st>>>(a);
    CK(cudaGetLastError());
    return 0;
}

int launch_q4r4_small(const Q4Args &a, int sms, cudaStream_t st) {
    if (a.I % 32 != 0 || a.I > MOTY_QROW_MAX || a.I <= 0) return moty_set_error(MOTY_CUDA_EARG, "q4r4: I=%d", a.I);
    if (a.O <= 0 || a.S <= 0) return 0;
    if (a.tiles) return launch_q4_t<4>(a, a.ntiles_max, sms, st);
    if (a.S == 1) return launch_q4_t<1>(a, 1, sms, st);
    if (a.S == 2) return launch_q4_t<2>(a, 1, sms, st);
    return launch_q4_t<4>(a, (a.S + 3) / 4, sms, st);
}

int q4r4_init_device() {
    CK(cudaFuncSetAttribute(q4r4_small_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    CK(cudaFuncSetAttribute(q4r4_small_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    CK(cudaFuncSetAttribute(q4r4_small_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    return 0;
}

// moty_matmul_q4r4_s (nn/matmul.c:424-432) cuts S tokens into tiles of 32; inside
// a tile the first (tile size / 4 * 4) tokens take the 4-token kernel and the
// rest the token-by-token kernel.  form[t] = 1 for the former.
__global__ void q4r4_forms_kernel(uint8_t *form, int S) {
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= S) return;
    int t0 = t / 32 * 32;
    int ns = S - t0 < 32 ? S - t0 : 32;
    form[t] = (t - t0) < ns / 4 * 4 ? 1 : 0;
}

int launch_q4r4_forms(uint8_t *form, int S, cudaStream_t st) {
    if (S <= 0) return 0;
    q4r4_forms_kernel<<<(S + 255) / 256, 256, 0, st>>>(form, S);
    CK(cudaGetLastError());
    return 0;
}
