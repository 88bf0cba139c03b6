"""A whole decoder step on the GPU (moty_b200.decoder.DenseDecoder, composed like engines/qwen.c:681-740, and
GemmaDecoder, composed like engines/gemma.c:453-497) against the same composition of the CPU oracle's functions: a
prompt, then greedy decoding, on small models of those shapes."""
import numpy as np
import pytest

from conftest import same_bits

pytestmark = pytest.mark.gpu


def _rmsnorm(x, w, eps):
    """moty_hw_rmsnorm_ref (hw/hw_ops.h:14-18), row by row."""
    out = np.empty_like(x)
    for s in range(x.shape[0]):
        ms = np.float64(0)
        for v in x[s].astype(np.float64):
            ms += v * v
        r = np.float32(1) / np.sqrt(np.float32(ms / x.shape[1]) + np.float32(eps), dtype=np.float32)
        out[s] = (x[s] * r) * w
    return out


class _OracleModel:
    def __init__(self, oracle, W, cfg, max_t):
        from oracle import AttnCache
        self.o, self.W, self.cfg = oracle, W, cfg
        self.caches = [AttnCache(cfg["H"], cfg["KV"], cfg["hd"], max_t, theta=1e6, eps=1e-6, qn=l["qn"], kn=l["kn"]) for l in W["layers"]]

    def step(self, ids, pos):
        o, W = self.o, self.W
        hq, hs = W["head"]
        x = np.stack([(hs[i] * np.float32(1.0)) * hq[i].astype(np.float32) for i in ids]).astype(np.float32)
        for l, cache in zip(W["layers"], self.caches):
            n = _rmsnorm(x, l["in_ln"], 1e-6)
            q, k, v = (o.matmul_q_s(n, *l[m]) for m in ("q", "k", "v"))
            ctx = o.attn_core(q, k, v, pos, cache)
            x = x + o.matmul_q_s(ctx, *l["o"])
            n = _rmsnorm(x, l["post_ln"], 1e-6)
            h = o.silu_mul(o.matmul_q_s(n, *l["gate"]), o.matmul_q_s(n, *l["up"]))
            x = x + o.matmul_q_s(h, *l["down"])
        last = _rmsnorm(x[-1:], W["final_norm"], 1e-6)
        lg = o.matmul_q_s(last, hq, hs)[0]
        return o.argmax(lg), lg


@pytest.mark.parametrize("O,I", [(4096, 1024), (640, 2048), (300, 4096), (1000, 112)])
def test_product_with_add_and_norm_inside(gpu, O, I):
    """y = W * rmsnorm(x + t) and xout = x + t in ONE launch (moty_cuda_mat_apply_addnorm_dev) against the two-launch
    route (add_rmsnorm_dev, then mat_apply_dev): the same bits, and x itself is left alone."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(O + I)
    q = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    m = gpu.Mat.i8(q, sc)
    x = rng.standard_normal((1, I)).astype(np.float32); t = rng.standard_normal((1, I)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, I).astype(np.float32)
    dx, dt, dg = (torch.from_numpy(a).cuda() for a in (x, t, g))
    x2 = dx.clone(); nrm = torch.empty_like(dx); xout = torch.zeros_like(dx)
    y1 = torch.empty((1, O), device="cuda"); y2 = torch.empty((1, O), device="cuda")
    torch.cuda.synchronize()
    sh = C.c_void_p(gpu.stream_handle(torch.cuda.current_stream()))
    L, p, eps = gpu.lib(), (lambda a: C.c_void_p(a.data_ptr())), C.c_float(1e-6)
    assert L.moty_cuda_mat_addnorm_supported(m.h) == 1
    assert L.moty_cuda_add_rmsnorm_dev(p(x2), p(dt), p(nrm), p(dg), 1, I, eps, sh) == 0
    assert L.moty_cuda_mat_apply_dev(m.h, p(y1), p(nrm), 1, sh) == 0
    assert L.moty_cuda_mat_apply_addnorm_dev(m.h, p(y2), p(dx), p(dt), p(xout), p(dg), eps, sh) == 0
    torch.cuda.synchronize()
    assert same_bits(y1.cpu().numpy(), y2.cpu().numpy())
    assert same_bits(x2.cpu().numpy(), xout.cpu().numpy()) and same_bits(dx.cpu().numpy(), x)
    assert L.moty_cuda_mat_apply_addnorm_dev(m.h, p(y2), p(dx), p(dt), p(dx), p(dg), eps, sh) != 0      # xout must not be x


def test_kernels_of_the_layer_glue(gpu):
    """RMS norm, residual add and embedding rows on device buffers against their definitions."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(2)
    S, D, V = 5, 1000, 77
    x = rng.standard_normal((S, D)).astype(np.float32); w = rng.uniform(0.5, 1.5, D).astype(np.float32)
    dx, dw = torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(); out = torch.empty_like(dx)
    torch.cuda.synchronize()
    sh = C.c_void_p(gpu.stream_handle(torch.cuda.current_stream()))
    L = gpu.lib()
    assert L.moty_cuda_rmsnorm_dev(C.c_void_p(out.data_ptr()), C.c_void_p(dx.data_ptr()), C.c_void_p(dw.data_ptr()), S, D, C.c_float(1e-6), sh) == 0
    ref = _rmsnorm(x, w, 1e-6)
    assert np.abs(out.cpu().numpy() - ref).max() <= 2e-7 * np.abs(ref).max()
    y = rng.standard_normal((S, D)).astype(np.float32); dy = torch.from_numpy(y).cuda()
    torch.cuda.synchronize()
    assert L.moty_cuda_add_dev(C.c_void_p(dy.data_ptr()), C.c_void_p(dx.data_ptr()), C.c_longlong(S * D), sh) == 0
    assert same_bits(dy.cpu().numpy(), y + x)
    # add + norm in one launch: the same bits as the two entries one after the other
    t2 = rng.standard_normal((S, D)).astype(np.float32); dt2 = torch.from_numpy(t2).cuda()
    a1, a2 = dy.clone(), dy.clone(); o1, o2 = torch.empty_like(dx), torch.empty_like(dx)
    torch.cuda.synchronize()
    P = lambda t: C.c_void_p(t.data_ptr())
    assert L.moty_cuda_add_dev(P(a1), P(dt2), C.c_longlong(S * D), sh) == 0
    assert L.moty_cuda_rmsnorm_dev(P(o1), P(a1), P(dw), S, D, C.c_float(1e-6), sh) == 0
    assert L.moty_cuda_add_rmsnorm_dev(P(a2), P(dt2), P(o2), P(dw), S, D, C.c_float(1e-6), sh) == 0
    assert same_bits(a1.cpu().numpy(), a2.cpu().numpy()) and same_bits(o1.cpu().numpy(), o2.cpu().numpy())
    q = rng.integers(-127, 128, (V, D), dtype=np.int8); qs = rng.uniform(0.001, 0.02, V).astype(np.float32)
    E = gpu.Mat.i8(q, qs)
    ids = np.array([3, 76, 0, 3, 41], np.int32); dids = torch.from_numpy(ids).cuda()
    torch.cuda.synchronize()
    assert L.moty_cuda_embed_rows_dev(E.h, C.c_void_p(out.data_ptr()), C.c_void_p(dids.data_ptr()), S, C.c_float(1.0), sh) == 0
    assert same_bits(out.cpu().numpy(), np.stack([(qs[i] * np.float32(1)) * q[i].astype(np.float32) for i in ids]))


def test_greedy_tokens_match_the_oracle(gpu, oracle):
    """A 3-layer model (hidden 256, 8 query / 4 KV heads of 32, FFN 512, vocabulary 1000, tied int8 head): a prompt of 9
    tokens and 24 greedy steps give the same token ids as the oracle's composition.  Every stage agrees with its oracle
    to 1e-6 or bit for bit, but an ulp before a row quantizer moves an int8 code, and a network of random weights
    amplifies that from layer to layer: the logits are compared at 3e-2 of their magnitude, the token ids exactly."""
    from moty_b200.decoder import DenseDecoder, DenseLayer
    rng = np.random.default_rng(7)
    cfg = dict(H=8, KV=4, hd=32); D, I, V, NL = 256, 512, 1000, 3
    mk = lambda O, K: (rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.0005, 0.0015, O).astype(np.float32))
    W = {"layers": [], "head": mk(V, D), "final_norm": np.ones(D, np.float32)}
    W["head"] = (W["head"][0], (W["head"][1] * 20).astype(np.float32))          # embedding rows of unit size
    for _ in range(NL):
        W["layers"].append(dict(q=mk(cfg["H"] * cfg["hd"], D), k=mk(cfg["KV"] * cfg["hd"], D), v=mk(cfg["KV"] * cfg["hd"], D),
                                o=mk(D, cfg["H"] * cfg["hd"]), gate=mk(I, D), up=mk(I, D), down=mk(D, I),
                                in_ln=np.ones(D, np.float32), post_ln=np.ones(D, np.float32),
                                qn=np.ones(cfg["hd"], np.float32), kn=np.ones(cfg["hd"], np.float32)))
    max_t = 64
    fuse = lambda l: gpu.Mat.i8(np.concatenate([l[m][0] for m in "qkv"]), np.concatenate([l[m][1] for m in "qkv"]))
    layers = [DenseLayer(*(gpu.Mat.i8(*l[m]) for m in ("q", "k", "v", "o", "gate", "up", "down")), l["in_ln"], l["post_ln"], l["qn"], l["kn"],
                         qkv=fuse(l) if i != 1 else None)                # one layer without the fused [q|k|v] matrix
              for i, l in enumerate(W["layers"])]
    # fold_addnorm: layer 2's add+norm rides in its [q|k|v] product (layer 1 has no fused matrix: the plain route)
    dec = DenseDecoder(layers, gpu.Mat.i8(*W["head"]), W["final_norm"], cfg["H"], cfg["KV"], cfg["hd"], max_t, fold_addnorm=True, fold_ffn=True)
    om = _OracleModel(oracle, W, cfg, max_t)
    prompt = rng.integers(0, V, 9).astype(np.int32)
    tg, lg = dec.step(prompt, 0, want_logits=True)
    to, lo = om.step(prompt, 0)
    assert np.abs(lg - lo).max() <= 3e-2 * np.abs(lo).max()
    assert tg == to
    pos, got, want = len(prompt), [tg], [to]
    for _ in range(24):
        tg, lg = dec.step([got[-1]], pos, want_logits=True)
        to, lo = om.step([want[-1]], pos)
        assert np.abs(lg - lo).max() <= 3e-2 * np.abs(lo).max(), pos
        got.append(tg); want.append(to); pos += 1
    assert got == want
    # the same steps from a CUDA graph captured once (the attention core reads its position from the device): same ids,
    # also when the graph is used a second time from another position
    assert dec.greedy_graph(got[0], len(prompt), 24) == got[1:]
    assert dec.greedy_graph(got[4], len(prompt) + 4, 10) == got[5:15]
    dec.close()


def test_greedy_tokens_match_with_routed_layers(gpu, oracle):
    """The same with routed layers in place of the dense FFN (8 experts, top-2, combined per token in selection order as
    engines/olmoe.c:219-244 does; the router logits come from an f32 router matrix): prompt of 6 tokens, 12 greedy steps."""
    from moty_b200.decoder import DenseDecoder, DenseLayer
    from oracle import AttnCache, Experts
    rng = np.random.default_rng(21)
    H, KV, hd, D, I, V, NL, E, K = 4, 4, 32, 128, 64, 500, 2, 8, 2
    mk = lambda O, Kk: (rng.integers(-127, 128, (O, Kk), dtype=np.int8), rng.uniform(0.0005, 0.0015, O).astype(np.float32))
    hq, hs = mk(V, D); hs = (hs * 20).astype(np.float32)
    ones = lambda n: np.ones(n, np.float32)
    Ls, layers = [], []
    for _ in range(NL):
        l = dict(q=mk(H * hd, D), k=mk(KV * hd, D), v=mk(KV * hd, D), o=mk(D, H * hd), R=(rng.standard_normal((E, D)) * 0.5).astype(np.float32))
        g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
        d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
        gs, us = (rng.uniform(0.0005, 0.0015, (E, I)).astype(np.float32) for _ in range(2))
        ds = rng.uniform(0.0005, 0.0015, (E, D)).astype(np.float32)
        l["ex"] = Experts(E, K, I, D, g, u, d, gs, us, ds)
        m = gpu.Moe(E, K, I, D)
        for e in range(E):
            m.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
        m.set_router(gpu.Mat.f32(l["R"]))
        Ls.append(l)
        layers.append(DenseLayer(*(gpu.Mat.i8(*l[k]) for k in "qkvo"), None, None, None, ones(D), ones(D), ones(hd), ones(hd), moe=m, norm_topk=0))
    max_t = 32
    dec = DenseDecoder(layers, gpu.Mat.i8(hq, hs), ones(D), H, KV, hd, max_t)
    caches = [AttnCache(H, KV, hd, max_t, qn=ones(hd), kn=ones(hd)) for _ in Ls]

    def ostep(ids, pos):
        x = np.stack([(hs[i] * np.float32(1.0)) * hq[i].astype(np.float32) for i in ids]).astype(np.float32)
        for l, cache in zip(Ls, caches):
            n = _rmsnorm(x, ones(D), 1e-6)
            q, k, v = (oracle.matmul_q_s(n, *l[m]) for m in "qkv")
            x = x + oracle.matmul_q_s(oracle.attn_core(q, k, v, pos, cache), *l["o"])
            n = _rmsnorm(x, ones(D), 1e-6)
            logits = (n.astype(np.float64) @ l["R"].astype(np.float64).T).astype(np.float32)
            x = x + oracle.olmoe_moe(l["ex"], n, logits, 0)[0]
        return oracle.argmax(oracle.matmul_q_s(_rmsnorm(x[-1:], ones(D), 1e-6), hq, hs)[0])

    prompt = rng.integers(0, V, 6).astype(np.int32)
    got, want = [dec.step(prompt, 0)], [ostep(prompt, 0)]
    for i in range(12):
        got.append(dec.step([got[-1]], 6 + i)); want.append(ostep([want[-1]], 6 + i))
    assert got == want
    assert dec.greedy_graph(got[0], 6, 12) == got[1:]
    dec.close()


@pytest.mark.parametrize("D,I,act,sandwich", [(3840, 1536, 1, True), (1024, 3072, 0, False), (2048, 520, 0, True), (112, 40, 1, False)])
def test_residual_and_norm_inside_the_consumers(gpu, D, I, act, sandwich):
    """The residual step (x + t, or gemma's x + rmsnorm(t) * g_t) and the norm that follows it, folded into the one-token
    product (moty_cuda_mat_apply_resnorm_dev) and into the FFN block (moty_cuda_ffn_resnorm_dev), against the separate
    entries one after the other: the same bits for y / out and for the new residual; x and t are left alone."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(D + I)
    mk = lambda O, K: gpu.Mat.i8(rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32))
    W, G, U, Dn = mk(I, D), mk(I, D), mk(I, D), mk(D, I)
    x, t = (rng.standard_normal((1, D)).astype(np.float32) for _ in range(2))
    gt, gx = (rng.uniform(0.5, 1.5, D).astype(np.float32) for _ in range(2))
    dx, dt, dgt, dgx = (torch.from_numpy(a).cuda() for a in (x, t, gt, gx))
    xs, nrm = dx.clone(), torch.empty_like(dx)
    y1, y2 = torch.empty((1, I), device="cuda"), torch.empty((1, I), device="cuda")
    o1, o2 = torch.empty_like(dx), torch.empty_like(dx)
    xo1, xo2 = torch.zeros_like(dx), torch.zeros_like(dx)
    torch.cuda.synchronize()
    sh = C.c_void_p(gpu.stream_handle(torch.cuda.current_stream()))
    L, P, eps = gpu.lib(), (lambda a: C.c_void_p(a.data_ptr())), C.c_float(1e-6)
    pgt = P(dgt) if sandwich else None
    if sandwich:
        assert L.moty_cuda_normadd_rmsnorm_dev(P(xs), P(dt), P(dgt), P(nrm), P(dgx), 1, D, eps, sh) == 0
    else:
        assert L.moty_cuda_add_rmsnorm_dev(P(xs), P(dt), P(nrm), P(dgx), 1, D, eps, sh) == 0
    assert L.moty_cuda_mat_apply_dev(W.h, P(y1), P(nrm), 1, sh) == 0
    assert L.moty_cuda_ffn_dev(G.h, U.h, Dn.h, act, P(o1), P(nrm), 1, sh) == 0
    assert L.moty_cuda_mat_addnorm_supported(W.h) == 1 and L.moty_cuda_ffn_resnorm_supported(G.h, U.h) == 1
    assert L.moty_cuda_mat_apply_resnorm_dev(W.h, P(y2), P(dx), P(dt), pgt, P(xo1), P(dgx), eps, sh) == 0, L.moty_cuda_last_error()
    assert L.moty_cuda_ffn_resnorm_dev(G.h, U.h, Dn.h, act, P(o2), P(dx), P(dt), pgt, P(xo2), P(dgx), eps, sh) == 0, L.moty_cuda_last_error()
    torch.cuda.synchronize()
    assert same_bits(y1.cpu().numpy(), y2.cpu().numpy()) and same_bits(o1.cpu().numpy(), o2.cpu().numpy())
    assert same_bits(xs.cpu().numpy(), xo1.cpu().numpy()) and same_bits(xs.cpu().numpy(), xo2.cpu().numpy())
    assert same_bits(dx.cpu().numpy(), x) and same_bits(dt.cpu().numpy(), t)
    assert L.moty_cuda_ffn_resnorm_dev(G.h, U.h, Dn.h, act, P(o2), P(dx), P(dt), pgt, P(dx), P(dgx), eps, sh) != 0       # xout must not be x


@pytest.mark.parametrize("D", [3840, 1000, 5000])
def test_sandwich_norm_step(gpu, D):
    """x += rmsnorm(t) * g1, out = rmsnorm(x) * g2 in one launch (moty_cuda_normadd_rmsnorm_dev) against the three
    entries one after the other: the same bits (rows held in registers up to 4096 values, re-read beyond)."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(D)
    S = 3
    x, t = (rng.standard_normal((S, D)).astype(np.float32) for _ in range(2))
    g1, g2 = (rng.uniform(0.5, 1.5, D).astype(np.float32) for _ in range(2))
    dx, dt, dg1, dg2 = (torch.from_numpy(a).cuda() for a in (x, t, g1, g2))
    x1, x2, x3 = dx.clone(), dx.clone(), dx.clone()
    tn, o1, o2 = torch.empty_like(dx), torch.empty_like(dx), torch.empty_like(dx)
    torch.cuda.synchronize()
    sh = C.c_void_p(gpu.stream_handle(torch.cuda.current_stream()))
    L, P, eps = gpu.lib(), (lambda a: C.c_void_p(a.data_ptr())), C.c_float(1e-6)
    assert L.moty_cuda_rmsnorm_dev(P(tn), P(dt), P(dg1), S, D, eps, sh) == 0
    assert L.moty_cuda_add_dev(P(x1), P(tn), C.c_longlong(S * D), sh) == 0
    assert L.moty_cuda_rmsnorm_dev(P(o1), P(x1), P(dg2), S, D, eps, sh) == 0
    assert L.moty_cuda_normadd_rmsnorm_dev(P(x2), P(dt), P(dg1), P(o2), P(dg2), S, D, eps, sh) == 0
    assert L.moty_cuda_normadd_rmsnorm_dev(P(x3), P(dt), P(dg1), None, None, S, D, eps, sh) == 0      # without the second norm
    torch.cuda.synchronize()
    assert same_bits(x1.cpu().numpy(), x2.cpu().numpy()) and same_bits(o1.cpu().numpy(), o2.cpu().numpy())
    assert same_bits(x1.cpu().numpy(), x3.cpu().numpy()) and same_bits(dt.cpu().numpy(), t)
    ref = x + _rmsnorm(t, g1, 1e-6)
    assert np.abs(x2.cpu().numpy() - ref).max() <= 4e-7 * np.abs(ref).max()


def test_gemma_greedy_tokens_match_the_oracle(gpu, oracle):
    """A 3-layer model shaped like the gemma engine's (hidden 256, 4 query heads; two sliding layers of 2 KV heads x 32
    with window 8 and theta 1e4, one global layer of 1 KV head x 64, theta 1e6, 8 rotated pairs; GeGLU FFN 512; four
    sandwich norms and q/k/v head norms with zero-centred weights; embedding rows scaled by sqrt(hidden)): a prompt of
    12 tokens (longer than the window) and 20 greedy steps give the oracle's token ids; logits at 3e-2 of their
    magnitude for the reason given for the qwen-shaped model above (the GeLU adds ~1e-7 of its own: tanhf)."""
    from moty_b200.decoder import GemmaDecoder, GemmaLayer
    from oracle import AttnCache
    rng = np.random.default_rng(11)
    H, D, I, V = 4, 256, 512, 900
    geo = [dict(KV=2, hd=32, theta=1e4, window=8, rot=16), dict(KV=2, hd=32, theta=1e4, window=8, rot=16),
           dict(KV=1, hd=64, theta=1e6, window=0, rot=8)]
    mk = lambda O, K: (rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.0005, 0.0015, O).astype(np.float32))
    w = lambda n: rng.uniform(-0.2, 0.2, n).astype(np.float32)             # zero-centred norm weights
    mult = lambda a: (np.float32(1) + a).astype(np.float32)
    hq, hs = mk(V, D); hs = (hs * 20 / 16).astype(np.float32)               # rows of unit size after the sqrt(256) scale
    fin = w(D)
    max_t = 48
    Ls, layers, caches = [], [], []
    for g in geo:
        qw, kw = H * g["hd"], g["KV"] * g["hd"]
        l = dict(q=mk(qw, D), k=mk(kw, D), v=mk(kw, D), o=mk(D, qw), gate=mk(I, D), up=mk(I, D), down=mk(D, I),
                 ln=[w(D) for _ in range(4)], qn=w(g["hd"]), kn=w(g["hd"]), vn=w(g["hd"]))
        Ls.append(l)
        fuse = gpu.Mat.i8(np.concatenate([l[m][0] for m in "qkv"]), np.concatenate([l[m][1] for m in "qkv"]))
        layers.append(GemmaLayer(*(gpu.Mat.i8(*l[m]) for m in ("q", "k", "v", "o", "gate", "up", "down")), *(mult(a) for a in l["ln"]),
                                 mult(l["qn"]), mult(l["kn"]), mult(l["vn"]), n_kv_heads=g["KV"], head_dim=g["hd"], theta=g["theta"],
                                 window=g["window"], rot=g["rot"], qkv=fuse if len(layers) != 1 else None))
        caches.append(AttnCache(H, g["KV"], g["hd"], max_t, theta=g["theta"], eps=1e-6, rot=g["rot"], qn=l["qn"], kn=l["kn"], vn=l["vn"],
                                gemma=True, window=g["window"]))
    dec = GemmaDecoder(layers, gpu.Mat.i8(hq, hs), mult(fin), H, max_t, fold_addnorm=True, fold_ffn=True)   # sandwich steps folded into their consumers
    es = np.sqrt(np.float32(D))

    def ostep(ids, pos):
        x = np.stack([(hs[i] * es) * hq[i].astype(np.float32) for i in ids]).astype(np.float32)
        for l, cache in zip(Ls, caches):
            n = _rmsnorm(x, mult(l["ln"][0]), 1e-6)
            q, k, v = (oracle.matmul_q_s(n, *l[m]) for m in "qkv")
            t = oracle.matmul_q_s(oracle.attn_core(q, k, v, pos, cache), *l["o"])
            x = x + _rmsnorm(t, mult(l["ln"][1]), 1e-6)
            n = _rmsnorm(x, mult(l["ln"][2]), 1e-6)
            h = oracle.gelu_mul(oracle.matmul_q_s(n, *l["gate"]), oracle.matmul_q_s(n, *l["up"]))
            x = x + _rmsnorm(oracle.matmul_q_s(h, *l["down"]), mult(l["ln"][3]), 1e-6)
        lg = oracle.matmul_q_s(_rmsnorm(x[-1:], mult(fin), 1e-6), hq, hs)[0]
        return oracle.argmax(lg), lg

    prompt = rng.integers(0, V, 12).astype(np.int32)
    tg, lg = dec.step(prompt, 0, want_logits=True)
    to, lo = ostep(prompt, 0)
    assert np.abs(lg - lo).max() <= 3e-2 * np.abs(lo).max()
    assert tg == to
    got, want, pos = [tg], [to], len(prompt)
    for _ in range(20):
        tg, lg = dec.step([got[-1]], pos, want_logits=True)
        to, lo = ostep([want[-1]], pos)
        assert np.abs(lg - lo).max() <= 3e-2 * np.abs(lo).max(), pos
        got.append(tg); want.append(to); pos += 1
    assert got == want
    assert dec.greedy_graph(got[0], len(prompt), 20) == got[1:]
    # the blocked prefill (blocks of 5 tokens) reaches the same first token
    assert dec.prefill(prompt, 0, block=5) == got[0]
    dec.close()
    # the same without the folds (every sandwich step its own launch): the same logits bit for bit
    plain = GemmaDecoder(layers, gpu.Mat.i8(hq, hs), mult(fin), H, max_t)
    dec2 = GemmaDecoder(layers, gpu.Mat.i8(hq, hs), mult(fin), H, max_t, fold_addnorm=True, fold_ffn=True)
    ta, la = plain.step(prompt, 0, want_logits=True); tb, lb = dec2.step(prompt, 0, want_logits=True)
    assert ta == tb and same_bits(la, lb)
    for i in range(4):
        ta, la = plain.step([ta], len(prompt) + i, want_logits=True); tb, lb = dec2.step([tb], len(prompt) + i, want_logits=True)
        assert ta == tb and same_bits(la, lb)
    plain.close(); dec2.close()
