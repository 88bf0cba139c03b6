// moe.cu -- device-side pieces of the FFN and MoE blocks: activation*up, the
// routing plan (token lists per expert and tile tables for the grouped
// products), the ordered weighted combine, and the f32 router GEMV.
#include "kernels.cuh"
#include "moe.cuh"

// ---------------------------------------------------------------------------
// g = act(g) * u.  SiLU: v / (1 + exp(-v)) (hw/hw_ops.h:19-21); tanh-GeLU:
// 0.5 v (1 + tanh(0.79788456 (v + 0.044715 v^3))) (engines/gemma.c:389-391).
// Both expressions live in common.cuh (moty_silu_mul, moty_gelu_mul), f32 step by f32 step.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) act_mul_kernel(float *__restrict__ g, const float *__restrict__ u, long long n, int act) {
    pdl_trigger();
    pdl_wait();
    long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    g[i] = act == MOTY_ACT_SILU ? moty_silu_mul(g[i], u[i]) : moty_gelu_mul(g[i], u[i]);
}

int launch_act_mul(float *g, const float *u, int64_t n, int act, cudaStream_t st) {
    if (n <= 0) return 0;
    CK(moty_launch_pdl(act_mul_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), (size_t)0, st, g, u, (long long)n, act));
    return 0;
}

// ---------------------------------------------------------------------------
// Routing plan.  Input: idx [S][K] (expert of every selection).  One CTA.
//   cnt/off per local expert, pairs sorted by (expert, token):
//     pair_tok[p]  token of position p          (gather map of the gate/up product)
//     pos_of[s*K+k] position of selection (s,k), -1 when its expert is not local
//   tile tables for the grouped products (tile = up to T positions of one expert)
//   ord[s*K + j]: the token's selections in combine order
//   form[p]: which of the two Q4R4 kernels the reference would use for that row
// ---------------------------------------------------------------------------
//
// The selections are cut into 32 contiguous segments, one per warp.  Pass A counts every
// segment's selections per expert (warp-private rows of a [32][E] table, lanes with the same
// expert found by match_any); a prefix over the warps turns the rows into each segment's first
// position inside the expert's list; pass B walks the segments again and hands out positions in
// ascending selection order, which keeps tokens ascending inside an expert (the order of the
// reference's gathered batches, nn/moe.c:172-186).
__global__ void __launch_bounds__(1024) moe_plan_kernel(MoePlanArgs a) {
    extern __shared__ int sh[];
    int *cnt = sh, *off = sh + a.E, *toff = sh + 2 * a.E, *wcnt = sh + 3 * a.E;      // [E], [E], [E], [32][E]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int SK = a.S * a.K, E = a.E;
    const int seg = ((SK + 31) / 32 + 31) / 32 * 32;                                 // selections per warp, a multiple of 32
    const int i_lo = warp * seg, i_hi = i_lo + seg < SK ? i_lo + seg : SK;
    pdl_trigger();
    pdl_wait();                                                                      // idx comes from the router launch
    for (int j = tid; j < 32 * E; j += 1024) wcnt[j] = 0;
    __syncthreads();
    for (int i0 = i_lo; i0 < i_hi; i0 += 32) {                                       // pass A
        const int i = i0 + lane;
        const int e = i < i_hi ? a.idx[i] : -1;
        const bool hit = e >= a.e_lo && e < a.e_hi;
        const unsigned m = __match_any_sync(0xffffffffu, hit ? e : -1 - lane);      // misses match nobody
        if (hit && (m & ((1u << lane) - 1u)) == 0) wcnt[warp * E + e] += __popc(m);  // lowest lane of each expert's set
        __syncwarp();
    }
    __syncthreads();
    for (int e = tid; e < E; e += 1024) {                                            // exclusive prefix over the warps
        int run = 0;
        for (int w = 0; w < 32; w++) { int t = wcnt[w * E + e]; wcnt[w * E + e] = run; run += t; }
        cnt[e] = run;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0, nt = 0;
        for (int e = 0; e < E; e++) { off[e] = run; toff[e] = nt; run += cnt[e]; nt += (cnt[e] + a.T - 1) / a.T; }
        *a.ntiles = nt;
        *a.npairs = run;
    }
    __syncthreads();
    for (int e = tid; e < E; e += 1024) {                                            // tile tables: up to T positions of one expert
        const int c = cnt[e], le = e - a.e_lo;
        int nt = toff[e];
        for (int r0 = 0; r0 < c; r0 += a.T, nt++) {
            const int nr = c - r0 < a.T ? c - r0 : a.T, row0 = off[e] + r0;
            if (a.q8) {
                a.t8_gate[nt] = Q8Tile{a.g8 + (size_t)le * a.gstride, a.gs + (size_t)le * a.gsstride, row0, nr};
                a.t8_up[nt]   = Q8Tile{a.u8 + (size_t)le * a.gstride, a.us + (size_t)le * a.gsstride, row0, nr};
                a.t8_down[nt] = Q8Tile{a.d8 + (size_t)le * a.dstride, a.ds + (size_t)le * a.dsstride, row0, nr};
            } else {
                a.t4_gate[nt] = Q4Tile{a.g4 + (size_t)le * a.gstride, a.gs16 + (size_t)le * a.gsstride, row0, nr};
                a.t4_up[nt]   = Q4Tile{a.u4 + (size_t)le * a.gstride, a.us16 + (size_t)le * a.gsstride, row0, nr};
                a.t4_down[nt] = Q4Tile{a.d4 + (size_t)le * a.dstride, a.ds16 + (size_t)le * a.dsstride, row0, nr};
            }
        }
    }
    for (int i0 = i_lo; i0 < i_hi; i0 += 32) {                                       // pass B
        const int i = i0 + lane;
        const int e = i < i_hi ? a.idx[i] : -1;
        const bool hit = e >= a.e_lo && e < a.e_hi;
        const unsigned m = __match_any_sync(0xffffffffu, hit ? e : -1 - lane);
        if (hit) {
            const int t = wcnt[warp * E + e] + __popc(m & ((1u << lane) - 1u));      // row inside this expert's gathered batch
            const int p = off[e] + t;
            a.pair_tok[p] = i / a.K;
            a.pos_of[i] = p;
            if (a.form) {
                const int c = cnt[e], t0 = t / 32 * 32, ns = c - t0 < 32 ? c - t0 : 32;
                a.form[p] = (t - t0) < ns / 4 * 4 ? 1 : 0;
            }
        } else if (i < i_hi) {
            a.pos_of[i] = -1;                                                        // selections of non-local experts
        }
        __syncwarp();
        if (hit && (m & ((1u << lane) - 1u)) == 0) wcnt[warp * E + e] += __popc(m);
        __syncwarp();
    }
    // combine order per token: the token's K expert ids are read once into local arrays and sorted there (the
    // insertion sort's dependent reads would otherwise each be a round trip to global memory)
    for (int s = tid; s < a.S; s += 1024) {
        int *o = a.ord + (size_t)s * a.K;
        if (a.order != 1) {
            for (int k = 0; k < a.K; k++) o[k] = k;
            continue;
        }
        int ix[64], ok[64];                              // K <= 64; ascending expert id, stable
        const int *src = a.idx + (size_t)s * a.K;
        for (int k = 0; k < a.K; k++) { ix[k] = src[k]; ok[k] = k; }
        for (int k = 1; k < a.K; k++) {
            const int v = ok[k], ve = ix[k];
            int j = k - 1;
            while (j >= 0 && ix[j] > ve) { ix[j + 1] = ix[j]; ok[j + 1] = ok[j]; j--; }
            ix[j + 1] = ve; ok[j + 1] = v;
        }
        for (int k = 0; k < a.K; k++) o[k] = ok[k];
    }
}

int launch_moe_plan(const MoePlanArgs &a, cudaStream_t st) {
    size_t smem = (size_t)(3 + 32) * a.E * sizeof(int);
    if (smem > 200 * 1024) return moty_set_error(MOTY_CUDA_ELIMIT, "moe plan: E=%d", a.E);
    if (smem > 48 * 1024) CK(cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(moty_launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), smem, st, a));
    return 0;
}

// ---------------------------------------------------------------------------
// out[s][d] = sum over the token's selections, IN ORDER, of w * h[pos][d], each
// step one fused multiply-add starting from 0 (nn/moe.c:146-149, 200-202,
// engines/olmoe.c:240).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_combine_kernel(float *__restrict__ out, const float *__restrict__ h,
                                                          const float *__restrict__ w, const int *__restrict__ pos_of,
                                                          const int *__restrict__ ord, int S, int K, int D) {
    // one CTA per token: the K (position, weight) pairs in combine order go to shared memory once, then every thread
    // requests the K rows' values of its columns together (up to 8 loads in flight) before the ordered chain
    __shared__ int p_s[64];
    __shared__ float w_s[64];
    const int s = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x < K) {
        const int k = ord[(size_t)s * K + threadIdx.x];
        p_s[threadIdx.x] = pos_of[(size_t)s * K + k];
        w_s[threadIdx.x] = w[(size_t)s * K + k];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += 256) {
        float acc = 0.f;
        for (int j0 = 0; j0 < K; j0 += 8) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int p = j0 + j < K ? p_s[j0 + j] : -1;
                v[j] = p >= 0 ? __ldcs(h + (size_t)p * D + d) : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (j0 + j < K && p_s[j0 + j] >= 0) acc = fmaf(w_s[j0 + j], v[j], acc);
        }
        out[(size_t)s * D + d] = acc;
    }
}

int launch_moe_combine(float *out, const float *h, const float *w, const int *pos_of, const int *ord,
                       int S, int K, int D, cudaStream_t st) {
    if (S <= 0) return 0;
    CK(moty_launch_pdl(moe_combine_kernel, dim3(S), dim3(256), (size_t)0, st, out, h, w, pos_of, ord, S, K, D));
    return 0;
}

// The same ordered combine for expert outputs laid out per selection, h[(s*K + k)][D]
// (what comes back from an expert-parallel exchange): one CTA per token; order 0 =
// selection order, 1 = ascending expert id.
__global__ void __launch_bounds__(256) moe_combine_sk_kernel(float *__restrict__ out, const float *__restrict__ h,
                                                             const float *__restrict__ w, const int *__restrict__ idx,
                                                             int K, int D, int order) {
    __shared__ int ord[64];
    __shared__ float ws[64];
    const int s = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x == 0) {
        for (int k = 0; k < K; k++) ord[k] = k;
        if (order == 1) {
            const int *ix = idx + (size_t)s * K;
            for (int k = 1; k < K; k++) {
                int v = ord[k], j = k - 1;
                while (j >= 0 && ix[ord[j]] > ix[v]) { ord[j + 1] = ord[j]; j--; }
                ord[j + 1] = v;
            }
        }
        for (int k = 0; k < K; k++) ws[k] = w[(size_t)s * K + k];
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += 256) {
        float acc = 0.f;
        for (int j = 0; j < K; j++) {
            int k = ord[j];
            acc = fmaf(ws[k], h[((size_t)s * K + k) * D + d], acc);
        }
        out[(size_t)s * D + d] = acc;
    }
}

int launch_moe_combine_sk(float *out, const float *h, const float *w, const int *idx,
                          int S, int K, int D, int order, cudaStream_t st) {
    if (S <= 0) return 0;
    CK(moty_launch_pdl(moe_combine_sk_kernel, dim3(S), dim3(256), (size_t)0, st, out, h, w, idx, K, D, order));
    return 0;
}


// ---------------------------------------------------------------------------
// Expert-parallel decode over peer memory: the exchange and the combine in one launch.
// Every rank's one-launch decode kernel has stored the rows of ITS experts into the row tables of ALL ranks
// (plain peer stores over NVLink).  This kernel, next on the rank's stream, (1) tells every peer "my rows of step
// `epoch` are written" -- a system-scope fence, then one release store per peer into that peer's flag word for this
// rank (each writer owns its word: no atomics, values only grow) -- and (2) waits until all ranks' words in the LOCAL
// flag array have reached `epoch`, then adds the K rows of the local table in selection order (nn/moe.c:146-149).
// The wait is BOUNDED: about a second of polling, after which the CTA sets the error word and writes nothing
// (moty_cuda_kernel_status reports it).  One rank per GPU only: a kernel that waits for another rank's kernel must
// never share a GPU with it.
// ---------------------------------------------------------------------------
constexpr unsigned PEER_WAIT_LIMIT = 1u << 21;

struct PeerCombineArgs {
    float *out; const float *table; const float *w; const int *idx;
    unsigned *flags_peer[8]; unsigned *flags_local;
    int K, D, world, rank; unsigned epoch; int *err;
};

__global__ void __launch_bounds__(256) moe_peer_combine_kernel(PeerCombineArgs a) {
    __shared__ float w_s[64];
    __shared__ int ok_s;
    if (threadIdx.x == 0) {
        ok_s = 1;
        if (blockIdx.x == 0) {
            __threadfence_system();                 // the decode kernel's peer stores (earlier on this stream) before the flags
            for (int r = 0; r < a.world; r++)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flags_peer[r] + a.rank), "r"(a.epoch) : "memory");
        }
        for (int r = 0; r < a.world && ok_s; r++) {
            unsigned n = 0, v;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(a.flags_local + r) : "memory");
                if ((int)(v - a.epoch) >= 0) break;                  // that rank has reached this step (or a later one)
                if (++n > PEER_WAIT_LIMIT) { ok_s = 0; break; }
            }
        }
        if (!ok_s) atomicExch(a.err, 1);
    }
    if (threadIdx.x < a.K) w_s[threadIdx.x] = a.w[threadIdx.x];
    __syncthreads();
    if (!ok_s) return;
    const int d = blockIdx.x * 256 + threadIdx.x;
    if (d >= a.D) return;
    float acc = 0.f;
    for (int k = 0; k < a.K; k++) acc = fmaf(w_s[k], __ldcv(a.table + (size_t)k * a.D + d), acc);   // peer-written: no stale cache line
    a.out[d] = acc;
}

int launch_moe_peer_combine(float *out, const float *table, const float *w, const int *idx, int K, int D,
                            unsigned *const *flags_peer, unsigned *flags_local, int world, int rank, unsigned epoch,
                            int *err, cudaStream_t st) {
    if (world < 1 || world > 8 || rank < 0 || rank >= world || K < 1 || K > 64)
        return moty_set_error(MOTY_CUDA_EARG, "moe_peer_combine: world=%d rank=%d K=%d", world, rank, K);
    PeerCombineArgs a;
    a.out = out; a.table = table; a.w = w; a.idx = idx; a.flags_local = flags_local;
    for (int r = 0; r < 8; r++) a.flags_peer[r] = r < world ? flags_peer[r] : nullptr;
    a.K = K; a.D = D; a.world = world; a.rank = rank; a.epoch = epoch; a.err = err;
    moe_peer_combine_kernel<<<(D + 255) / 256, 256, 0, st>>>(a);
    CK(cudaGetLastError());
    return 0;
}

// ---------------------------------------------------------------------------
// f32 matrix (router of an engine that keeps it unquantized): one warp per
// output row, f32 accumulation.  Outside the quantized path; the summation
// order differs from a CPU SIMD dot, so it is close, not bit-equal.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) f32_rows_kernel(const float *__restrict__ W, const float *__restrict__ x,
                                                       float *__restrict__ y, int S, int I, int O) {
    // a warp takes one output row and four consecutive tokens (blockIdx.y); per (row, token) the same lane-strided
    // fmaf chain and shuffle tree whatever the batch size, so a token's logits do not depend on how many come with it
    // (the loads of sixteen steps of the chain are requested together and the weight row is read once for the four
    // tokens; the chain itself is the plain one: a layer's router is a launch of its own in front of the experts, and with
    // one load in flight per lane it took 17 us for 128 x 2048)
    int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (o >= O) return;
    const int s0 = blockIdx.y * 4, nt = S - s0 < 4 ? S - s0 : 4;
    const float *wr = W + (size_t)o * I, *xr = x + (size_t)s0 * I;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    int i = lane;
    for (; i + 15 * 32 < I; i += 16 * 32) {
        float wv[16];
#pragma unroll
        for (int u = 0; u < 16; u++) wv[u] = __ldg(wr + i + 32 * u);
#pragma unroll
        for (int t = 0; t < 4; t++) {
            if (t >= nt) break;
            float xv[16];
#pragma unroll
            for (int u = 0; u < 16; u++) xv[u] = xr[(size_t)t * I + i + 32 * u];
#pragma unroll
            for (int u = 0; u < 16; u++) acc[t] = fmaf(wv[u], xv[u], acc[t]);
        }
    }
    for (; i < I; i += 32) {
        const float wv = __ldg(wr + i);
#pragma unroll
        for (int t = 0; t < 4; t++) if (t < nt) acc[t] = fmaf(wv, xr[(size_t)t * I + i], acc[t]);
    }
#pragma unroll
    for (int t = 0; t < 4; t++) {
        if (t >= nt) break;
        float a = acc[t];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) a += __shfl_xor_sync(0xffffffffu, a, d);
        if (lane == 0) y[(size_t)(s0 + t) * O + o] = a;
    }
}

int launch_f32_rows(const float *W, const float *x, float *y, int S, int I, int O, cudaStream_t st) {
    if (O <= 0 || S <= 0) return 0;
    // a plain launch on purpose: chained programmatically it measured slower over a whole OLMoE-shaped decode step, with
    // the cooperative layer kernel after it (1095 against 1116 tok/s replayed) and with the two chained layer launches
    // (1129 against 1217; same GPU, twice each); again after the loads were batched, with the first weights requested
    // before the wait: 1272 against 1323 tok/s on that shape, 424 against 421 on the Qwen3-30B-A3B shape
    if ((S + 3) / 4 > 65535) return moty_set_error(MOTY_CUDA_ELIMIT, "f32 matrix: S=%d in one call", S);
    f32_rows_kernel<<<dim3((O + 7) / 8, (S + 3) / 4), 256, 0, st>>>(W, x, y, S, I, O);
    CK(cudaGetLastError());
    return 0;
}
