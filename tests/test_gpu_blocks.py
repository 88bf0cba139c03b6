"""GPU parity of the FFN and MoE blocks through the C ABI."""
import numpy as np
import pytest

from conftest import golden, same_bits

pytestmark = pytest.mark.gpu

# SiLU blocks (FFN, MoE) are compared BIT FOR BIT with the reference: the library evaluates expf by
# the C library's own algorithm (moty_expf), every other step is a correctly rounded f32 operation in
# the reference's order.  Only the tanh-GeLU block keeps a tolerance: tanhf is the C library's
# float routine, which is not restated, and one ulp before the re-quantization of the hidden row can
# move an int8 code by one (1/127 of one term); it is bit-exact whenever the hidden codes agree.
TOL = 1e-5


def close(a, b, tol=TOL):
    scale = max(float(np.abs(b).max()), 1e-30)
    return float(np.abs(a - b).max()) <= tol * scale


def test_ffn_q8_and_q4r4(gpu, oracle):
    g = golden("blocks")
    G = gpu.Mat.i8(g["gq"], g["gs"]); U = gpu.Mat.i8(g["uq"], g["us"]); Dn = gpu.Mat.i8(g["dq"], g["ds"])
    G4 = gpu.Mat.q4r4(g["g4"], g["g4s"], 256, 128); U4 = gpu.Mat.q4r4(g["u4"], g["u4s"], 256, 128)
    D4 = gpu.Mat.q4r4(g["d4"], g["d4s"], 128, 256)
    for S in (1, 5):
        x = g[f"ffn_x{S}"]
        assert same_bits(gpu.dense_ffn(G, U, Dn, x), g[f"ffn8_{S}"])
        assert same_bits(gpu.dense_ffn(G4, U4, D4, x), g[f"ffn4_{S}"])
        y = gpu.dense_ffn(G, U, Dn, x, act=gpu.ACT_GELU_TANH)
        h = oracle.gelu_mul(oracle.matmul_q_s(x, g["gq"], g["gs"]), oracle.matmul_q_s(x, g["uq"], g["us"]))
        yo = oracle.matmul_q_s(h, g["dq"], g["ds"])
        # tanh-GeLU: the C library's tanhf is not restated (the GPU rounds tanh once from f64), so a hidden value can differ
        # by an ulp and move one int8 code of the re-quantized row: rows whose codes agree come out bit for bit, the others
        # differ by 1/127 of one term
        exact = int(sum(y[r].tobytes() == yo[r].tobytes() for r in range(S)))
        print(f"GeLU FFN S={S}: {exact} of {S} output rows bit-identical to the CPU reference's arithmetic")
        assert close(y, yo, 2e-3)


@pytest.mark.parametrize("D,I", [(1024, 3072), (2048, 4096), (1008, 2064), (64, 48)])
def test_ffn_decode_one_launch_equals_steps(gpu, oracle, D, I):
    """One token, int8 matrices, SiLU: the default route (gate + up + activation in one launch, then the down product), the
    one-launch cooperative kernel that runs the block as a one-expert MoE decode block (fast path 3) and the step-by-step
    path (gate, up, activation, down) give the same bits, and those of the oracle."""
    rng = np.random.default_rng(D + I)
    mk = lambda O, K: (rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32))
    (gq, gs), (uq, us), (dq, ds) = mk(I, D), mk(I, D), mk(D, I)
    G, U, Dn = gpu.Mat.i8(gq, gs), gpu.Mat.i8(uq, us), gpu.Mat.i8(dq, ds)
    for _ in range(2):                                  # twice: the grid barrier's words have to be back at zero
        x = rng.standard_normal((1, D)).astype(np.float32)
        prev = gpu.lib().moty_cuda_set_moe_fast_path(1)
        y1 = gpu.dense_ffn(G, U, Dn, x)
        gpu.lib().moty_cuda_set_moe_fast_path(3)
        y3 = gpu.dense_ffn(G, U, Dn, x)
        gpu.lib().moty_cuda_set_moe_fast_path(0)
        y0 = gpu.dense_ffn(G, U, Dn, x)
        gpu.lib().moty_cuda_set_moe_fast_path(prev)
        assert same_bits(y1, y0) and same_bits(y3, y0)
        h = oracle.silu_mul(oracle.matmul_q_s(x, gq, gs), oracle.matmul_q_s(x, uq, us))
        assert same_bits(y1, oracle.matmul_q_s(h, dq, ds))


@pytest.mark.parametrize("D,I,act", [(3840, 1536, 1), (2560, 5000, 0), (1024, 3072, 1), (4096, 520, 0), (48, 40, 1)])
def test_ffn_decode_gate_up_in_one_launch(gpu, oracle, D, I, act):
    """One token, int8 matrices, tanh-GeLU and SiLU, sizes up to rows of 4096 values (the gemma block's 3840 among them):
    gate, up and the activation run as one launch (q8_gateup_kernel), then the down product.  The output equals the
    step-by-step path bit for bit, and -- with SiLU -- the oracle bit for bit (GeLU: see test_ffn_q8_and_q4r4)."""
    rng = np.random.default_rng(D + I + act)
    mk = lambda O, K: (rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32))
    (gq, gs), (uq, us), (dq, ds) = mk(I, D), mk(I, D), mk(D, I)
    G, U, Dn = gpu.Mat.i8(gq, gs), gpu.Mat.i8(uq, us), gpu.Mat.i8(dq, ds)
    x = rng.standard_normal((1, D)).astype(np.float32)
    prev = gpu.lib().moty_cuda_set_moe_fast_path(1)
    y1 = gpu.dense_ffn(G, U, Dn, x, act=act)
    gpu.lib().moty_cuda_set_moe_fast_path(0)
    y0 = gpu.dense_ffn(G, U, Dn, x, act=act)
    gpu.lib().moty_cuda_set_moe_fast_path(prev)
    assert same_bits(y1, y0)
    gx, ux = oracle.matmul_q_s(x, gq, gs), oracle.matmul_q_s(x, uq, us)
    yo = oracle.matmul_q_s(oracle.silu_mul(gx, ux) if act == 0 else oracle.gelu_mul(gx, ux), dq, ds)
    assert same_bits(y1, yo) if act == 0 else close(y1, yo, 2e-3)


def test_attn_core_golden(gpu):
    """Attention core on the GPU against the vectors composed from the reference's functions: three calls per case
    (a prompt of 5, one decode step, 3 more tokens) on one cache; f32 and int8 KV, QK-norm on and off, partial rotary.
    f32 sums in another order and libm against CUDA's powf/cosf/sinf/expf: 5e-5 of the output magnitude (2e-3 with
    the int8 cache, where an ulp before the row quantizer can move a code)."""
    from test_oracle import _attn_golden_cases
    g = golden("attn")
    for tag, _, steps in _attn_golden_cases():
        H, KV, hd, rot, norm, kv8 = (int(v) for v in g[f"cfg_{tag}"])
        a = gpu.Attn(H, KV, hd, 16, theta=1e6, eps=1e-6, rot=rot, qn=g[f"qn_{tag}"] if norm else None,
                     kn=g[f"kn_{tag}"] if norm else None, kv8=bool(kv8))
        pos = 0
        for q, k, v, ctx in steps:
            y = a.core(q, k, v, pos)
            assert np.abs(y - ctx).max() <= (2e-3 if kv8 else 5e-5) * np.abs(ctx).max(), (tag, pos, float(np.abs(y - ctx).max()))
            pos += q.shape[0]
        a.close()


@pytest.mark.parametrize("H,KV,hd,rot,kv8", [(16, 8, 128, 128, False), (16, 8, 128, 128, True), (8, 4, 256, 128, False),
                                              (14, 2, 64, 64, True), (5, 5, 80, 40, False)])
def test_attn_core_vs_oracle(gpu, oracle, H, KV, hd, rot, kv8):
    """Model-sized heads and longer contexts: a prompt of 300 tokens, then decode steps, on one cache; grouped-query
    ratios 1..7, head sizes that are not powers of two, positions past 2048 (large RoPE angles)."""
    from oracle import AttnCache
    rng = np.random.default_rng(H * 3 + hd + int(kv8))
    qn = rng.uniform(0.5, 1.5, hd).astype(np.float32); kn = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    max_t = 2400
    cache = AttnCache(H, KV, hd, max_t, theta=1e6, eps=1e-6, rot=rot, qn=qn, kn=kn, kv8=kv8)
    a = gpu.Attn(H, KV, hd, max_t, theta=1e6, eps=1e-6, rot=rot, qn=qn, kn=kn, kv8=kv8)
    pos = 2050
    # positions below pos_base are zero rows in both caches: they take part in the softmax identically
    for S in (300, 1, 1, 17):
        q = rng.standard_normal((S, H * hd)).astype(np.float32)
        k = rng.standard_normal((S, KV * hd)).astype(np.float32); v = rng.standard_normal((S, KV * hd)).astype(np.float32)
        yo = oracle.attn_core(q.copy(), k.copy(), v.copy(), pos, cache)
        y = a.core(q, k, v, pos)
        # int8 cache: an ulp of difference before the row quantizer can move a code by one (1/127 of one term)
        tol = 2e-3 if kv8 else 5e-5
        err, mag = float(np.abs(y - yo).max()), float(np.abs(yo).max())
        print(f"attn H={H} hd={hd} kv8={kv8} S={S} pos={pos}: max err {err:.3g} of {mag:.3g}")
        assert err <= tol * mag, (S, pos, err, mag)
        pos += S
    a.close()
    with pytest.raises(RuntimeError):
        gpu.Attn(H, KV, hd, 8).core(np.zeros((9, H * hd), np.float32), np.zeros((9, KV * hd), np.float32),
                                    np.zeros((9, KV * hd), np.float32), 0)


@pytest.mark.parametrize("H,KV,hd,rot,kv8,T0,gemma", [(16, 8, 128, 128, False, 700, 0), (16, 8, 128, 128, True, 700, 0), (8, 2, 64, 32, False, 40, 0),
                                                       (4, 4, 256, 256, False, 300, 0), (12, 2, 96, 96, True, 1500, 0), (16, 2, 128, 64, False, 5, 0),
                                                       (16, 8, 256, 128, False, 1300, 1024), (16, 8, 256, 32, False, 900, -1), (4, 2, 64, 32, True, 50, 16)])
def test_attn_decode_one_launch_equals_two(gpu, H, KV, hd, rot, kv8, T0, gemma):
    """One token at a position read from the device: norm, rotation and cache store inside the scores launch.  Same
    context rows and same cache rows as the prep + scores pair of attn_core_dev, step after step (the f64 sum of squares
    is taken in another order, hence 1e-6 and not bit for bit), and q, k stay as they came.  gemma != 0: the gemma
    flavour (rot = rotated pairs, (1 + w) multipliers, value norm; > 0 = the sliding window, -1 = a global layer)."""
    import torch
    rng = np.random.default_rng(H * 1000 + hd + T0)
    max_t = T0 + 8
    qn = rng.uniform(0.5, 1.5, hd).astype(np.float32); kn = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    kw = dict(gemma=True, window=max(gemma, 0), vn=rng.uniform(0.5, 1.5, hd).astype(np.float32), theta=1e4) if gemma else {}
    a = gpu.Attn(H, KV, hd, max_t, rot=rot, qn=qn, kn=kn, kv8=kv8, **kw)
    b = gpu.Attn(H, KV, hd, max_t, rot=rot, qn=qn, kn=kn, kv8=kv8, **kw)
    f = lambda *sh: rng.standard_normal(sh).astype(np.float32)
    q0, k0, v0 = f(T0, H * hd), f(T0, KV * hd), f(T0, KV * hd)
    a.core(q0.copy(), k0.copy(), v0, 0); b.core(q0.copy(), k0.copy(), v0, 0)        # the same prompt in both caches
    sh = gpu.stream_handle(torch.cuda.current_stream())
    pos_dev = torch.zeros((1,), dtype=torch.int32, device="cuda")
    tol = 2e-3 if kv8 else 2e-6
    for step in range(6):
        q, k, v = f(1, H * hd), f(1, KV * hd), f(1, KV * hd)
        da = [torch.from_numpy(t.copy()).cuda() for t in (q, k, v)]
        db = [torch.from_numpy(t.copy()).cuda() for t in (q, k, v)]
        ca = torch.empty((1, H * hd), device="cuda"); cb = torch.empty((1, H * hd), device="cuda")
        pos_dev.fill_(T0 + step)
        a.core_dev(ca.data_ptr(), da[0].data_ptr(), da[1].data_ptr(), da[2].data_ptr(), 1, T0 + step, stream=sh)
        b.core_posdev(cb.data_ptr(), db[0].data_ptr(), db[1].data_ptr(), db[2].data_ptr(), 1, pos_dev.data_ptr(), max_t - 1, stream=sh)
        torch.cuda.synchronize()
        ya, yb = ca.cpu().numpy(), cb.cpu().numpy()
        assert np.isfinite(yb).all() and np.abs(ya - yb).max() <= tol * np.abs(ya).max(), (step, np.abs(ya - yb).max())
        assert np.array_equal(db[0].cpu().numpy(), q) and np.array_equal(db[1].cpu().numpy(), k)
    a.close(); b.close()


def test_attn_gate_and_device_entry(gpu, oracle):
    """The device-pointer entry on torch buffers (q and k are normed and rotated in place, as the reference does) and
    the gated variant's last step, ctx *= 1 / (1 + expf(-gate)) (nn/attn.c:68-69)."""
    import torch
    from oracle import AttnCache
    H, KV, hd, S = 8, 4, 64, 5
    rng = np.random.default_rng(11)
    qn = rng.uniform(0.5, 1.5, hd).astype(np.float32); kn = rng.uniform(0.5, 1.5, hd).astype(np.float32)
    q = rng.standard_normal((S, H * hd)).astype(np.float32); k = rng.standard_normal((S, KV * hd)).astype(np.float32)
    v = rng.standard_normal((S, KV * hd)).astype(np.float32); gate = rng.standard_normal((S, H * hd)).astype(np.float32)
    qo, ko = q.copy(), k.copy()
    yo = oracle.attn_core(qo, ko, v.copy(), 3, AttnCache(H, KV, hd, 16, qn=qn, kn=kn))
    a = gpu.Attn(H, KV, hd, 16, qn=qn, kn=kn)
    dq, dk, dv, dg = (torch.from_numpy(t).cuda() for t in (q, k, v, gate))
    ctx = torch.empty((S, H * hd), device="cuda")
    torch.cuda.synchronize()
    sh = gpu.stream_handle(torch.cuda.current_stream())
    a.core_dev(ctx.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), S, 3, stream=sh)
    torch.cuda.synchronize()
    assert np.abs(ctx.cpu().numpy() - yo).max() <= 5e-5 * np.abs(yo).max()
    assert np.abs(dq.cpu().numpy() - qo).max() <= 1e-5 and np.abs(dk.cpu().numpy() - ko).max() <= 1e-5
    a.gate_dev(ctx.data_ptr(), dg.data_ptr(), S, stream=sh)
    torch.cuda.synchronize()
    yg = yo * (np.float32(1) / (np.float32(1) + np.exp(-gate, dtype=np.float32)))
    assert np.abs(ctx.cpu().numpy() - yg).max() <= 5e-5 * np.abs(yg).max()
    a.close()


def _moe_from_golden(gpu, g):
    E, K, I, D = (int(v) for v in g["moe_dims"])
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert(e, g["moe_g"][e], g["moe_gs"][e], g["moe_u"][e], g["moe_us"][e], g["moe_d"][e], g["moe_ds"][e])
    return m


def test_moe_blocks_golden(gpu):
    g = golden("blocks")
    m = _moe_from_golden(gpu, g)
    assert same_bits(m.d1(g["moe_x1"], g["moe_logits1"]), g["moe_out1"])
    assert same_bits(m.batch(g["moe_x9"], g["moe_logits9"]), g["moe_out9"])
    for S in (1, 9):
        assert same_bits(m.olmoe(g[f"moe_x{S}"], g[f"moe_logits{S}"], 0), g[f"olmoe_out{S}"])
    # with the router on the GPU as an int8 matrix: same logits bit for bit -> same routing
    m.set_router(gpu.Mat.i8(g["moe_rq"], g["moe_rs"]))
    assert same_bits(m.d1(g["moe_x1"]), g["moe_out1"])
    assert same_bits(m.batch(g["moe_x9"]), g["moe_out9"])


@pytest.mark.parametrize("E,K,I,D,S", [(64, 8, 128, 256, 1), (64, 8, 128, 256, 40), (16, 4, 96, 160, 7)])
def test_moe_q8_vs_oracle(gpu, oracle, E, K, I, D, S):
    from oracle import Experts
    rng = np.random.default_rng(E + K + S)
    g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
    d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
    gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
    ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
    ex = Experts(E, K, I, D, g, u, d, gs, us, ds)
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
    x = rng.standard_normal((S, D)).astype(np.float32)
    logits = (rng.standard_normal((S, E)) * 0.5).astype(np.float32)
    want = (oracle.moe_d1 if S == 1 else oracle.moe_batch)(ex, x, logits)[0]
    got = m.d1(x, logits) if S == 1 else m.batch(x, logits)
    assert same_bits(got, want)
    want, idx, w = oracle.olmoe_moe(ex, x, logits, 0)
    assert same_bits(m.olmoe(x, logits, 0), want)


@pytest.mark.parametrize("S", [1, 3, 21, 80, 130])        # 80 and 130: 16- and 32-row tiles of the grouped MMA kernel
def test_moe_q4r4_vs_oracle(gpu, oracle, S):
    from oracle import Experts
    E, K, I, D = 16, 4, 96, 128
    rng = np.random.default_rng(S)
    packs = {k: [oracle.pack_q4r4((rng.standard_normal(shape) * 0.05).astype(np.float32)) for _ in range(E)]
             for k, shape in (("g", (I, D)), ("u", (I, D)), ("d", (D, I)))}
    cat = lambda k, j: np.concatenate([p[j] for p in packs[k]])
    ex = Experts(E, K, I, D, cat("g", 0), cat("u", 0), cat("d", 0), cat("g", 1), cat("u", 1), cat("d", 1))
    m = gpu.Moe(E, K, I, D, efmt=gpu.WF_Q4R4)
    for e in range(E):
        m.upload_expert(e, packs["g"][e][0], packs["g"][e][1], packs["u"][e][0], packs["u"][e][1],
                        packs["d"][e][0], packs["d"][e][1])
    x = rng.standard_normal((S, D)).astype(np.float32)
    logits = (rng.standard_normal((S, E)) * 0.5).astype(np.float32)
    want = oracle.moe_q4r4(ex, x, logits)[0]
    got = m.d1(x, logits) if S == 1 else m.batch(x, logits)
    assert same_bits(got, want)


@pytest.mark.parametrize("S", [21, 130])
def test_moe_q4r4_batch_relaxed(gpu, oracle, S):
    """A routed Q4R4 prompt with moty_cuda_set_q4r4_batch_relaxed(1): within 1e-5 of the oracle's magnitude per token
    (the grouped products use one formula for a group's term instead of the reference's two); the default is bit-exact
    before and after."""
    from oracle import Experts
    E, K, I, D = 16, 4, 96, 128
    rng = np.random.default_rng(100 + S)
    packs = {k: [oracle.pack_q4r4((rng.standard_normal(shape) * 0.05).astype(np.float32)) for _ in range(E)]
             for k, shape in (("g", (I, D)), ("u", (I, D)), ("d", (D, I)))}
    cat = lambda k, j: np.concatenate([p[j] for p in packs[k]])
    ex = Experts(E, K, I, D, cat("g", 0), cat("u", 0), cat("d", 0), cat("g", 1), cat("u", 1), cat("d", 1))
    m = gpu.Moe(E, K, I, D, efmt=gpu.WF_Q4R4)
    for e in range(E):
        m.upload_expert(e, packs["g"][e][0], packs["g"][e][1], packs["u"][e][0], packs["u"][e][1],
                        packs["d"][e][0], packs["d"][e][1])
    x = rng.standard_normal((S, D)).astype(np.float32)
    logits = (rng.standard_normal((S, E)) * 0.5).astype(np.float32)
    want = oracle.moe_q4r4(ex, x, logits)[0]
    assert same_bits(m.batch(x, logits), want)
    L = gpu.lib()
    prev = L.moty_cuda_set_q4r4_batch_relaxed(1)
    try:
        got = m.batch(x, logits)
    finally:
        L.moty_cuda_set_q4r4_batch_relaxed(prev)
    err = np.abs(got - want).max(axis=1) / np.abs(want).max(axis=1)
    assert err.max() <= 1e-5, err.max()
    assert same_bits(m.batch(x, logits), want)


def test_expert_shards_sum_to_the_whole(gpu, oracle):
    """Two expert-parallel shards: their partial outputs add up to the unsharded
    block (f32 sums in another order: compared at 1e-5 of magnitude)."""
    g = golden("blocks")
    E, K, I, D = (int(v) for v in g["moe_dims"])
    whole = _moe_from_golden(gpu, g).batch(g["moe_x9"], g["moe_logits9"])
    total = np.zeros_like(whole)
    for lo, hi in ((0, 4), (4, 8)):
        m = gpu.Moe(E, K, I, D, e_lo=lo, e_hi=hi)
        for e in range(lo, hi):
            m.upload_expert(e, g["moe_g"][e], g["moe_gs"][e], g["moe_u"][e], g["moe_us"][e], g["moe_d"][e], g["moe_ds"][e])
        total += m.batch(g["moe_x9"], g["moe_logits9"])
    assert close(total, whole)


@pytest.mark.parametrize("E,K,I,D,lo,hi", [(64, 8, 1024, 2048, 0, 64), (16, 4, 96, 160, 0, 16), (16, 4, 96, 160, 4, 12),
                                           (8, 8, 48, 2048, 0, 8), (32, 6, 2064, 512, 0, 32), (12, 10, 4096, 64, 0, 12)])
def test_moe_decode_fast_path_equals_generic_path(gpu, oracle, E, K, I, D, lo, hi):
    """The default decode path (1: route + gate/up, then down, two chained launches), the split decode path (2: a router
    launch first), the one-launch cooperative kernel (3) and the grouped path (0) are the same arithmetic: bit-identical,
    also on an expert shard (non-resident experts contribute nothing), and repeated calls keep the cooperative kernel's
    grid barrier consistent."""
    from oracle import Experts
    rng = np.random.default_rng(E * K + I + lo)
    g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
    d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
    gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
    ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
    m = gpu.Moe(E, K, I, D, e_lo=lo, e_hi=hi)
    for e in range(lo, hi):
        m.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
    for trial in range(3):
        x = rng.standard_normal((1, D)).astype(np.float32)
        logits = (rng.standard_normal((1, E)) * 0.5).astype(np.float32)
        prev = gpu.lib().moty_cuda_set_moe_fast_path(1)
        fast = m.d1(x, logits); fast_ol = m.olmoe(x, logits, 0)
        gpu.lib().moty_cuda_set_moe_fast_path(2)
        split = m.d1(x, logits); split_ol = m.olmoe(x, logits, 0)
        gpu.lib().moty_cuda_set_moe_fast_path(3)
        coop = m.d1(x, logits); coop_ol = m.olmoe(x, logits, 0)
        gpu.lib().moty_cuda_set_moe_fast_path(0)
        slow = m.d1(x, logits); slow_ol = m.olmoe(x, logits, 0)
        gpu.lib().moty_cuda_set_moe_fast_path(prev)
        assert same_bits(fast, slow) and same_bits(fast_ol, slow_ol)
        assert same_bits(split, slow) and same_bits(split_ol, slow_ol)
        assert same_bits(coop, slow) and same_bits(coop_ol, slow_ol)
    if (lo, hi) == (0, E):
        want = oracle.moe_d1(Experts(E, K, I, D, g, u, d, gs, us, ds), x, logits)[0]
        assert same_bits(fast, want)


@pytest.mark.parametrize("E,K,I,D,lo,hi", [(16, 4, 96, 128, 0, 16), (128, 8, 768, 2048, 0, 128), (16, 4, 96, 128, 8, 16),
                                           (16, 6, 1312, 416, 0, 16), (16, 4, 96, 128, 15, 16)])
def test_moe_q4r4_decode_fast_path_equals_generic_path(gpu, oracle, E, K, I, D, lo, hi):
    from oracle import Experts
    rng = np.random.default_rng(E + I + lo)
    small = E <= 16
    if small:
        packs = {k: [oracle.pack_q4r4((rng.standard_normal(shape) * 0.05).astype(np.float32)) for _ in range(E)]
                 for k, shape in (("g", (I, D)), ("u", (I, D)), ("d", (D, I)))}
    else:                                      # random codes and f16 scales: packing 128 experts on the CPU is slow
        ng, nd = (I // 4) * (D // 32), (D // 4) * (I // 32)
        mk = lambda n: (rng.integers(0, 256, n * 64, dtype=np.uint8),
                        rng.uniform(0.001, 0.01, n * 4).astype(np.float16).view(np.uint16))
        packs = {"g": [mk(ng) for _ in range(E)], "u": [mk(ng) for _ in range(E)], "d": [mk(nd) for _ in range(E)]}
    m = gpu.Moe(E, K, I, D, efmt=gpu.WF_Q4R4, e_lo=lo, e_hi=hi)
    for e in range(lo, hi):
        m.upload_expert(e, packs["g"][e][0], packs["g"][e][1], packs["u"][e][0], packs["u"][e][1],
                        packs["d"][e][0], packs["d"][e][1])
    for trial in range(3):
        x = rng.standard_normal((1, D)).astype(np.float32)
        logits = (rng.standard_normal((1, E)) * 0.5).astype(np.float32)
        prev = gpu.lib().moty_cuda_set_moe_fast_path(1)
        fast = m.d1(x, logits); fast2 = m.d1(x, logits)        # twice: the fused kernel's counters must come back to zero
        gpu.lib().moty_cuda_set_moe_fast_path(2)
        split = m.d1(x, logits)
        gpu.lib().moty_cuda_set_moe_fast_path(3)                # the one-launch cooperative form of the default's two chained launches
        coop = m.d1(x, logits); coop2 = m.d1(x, logits)
        gpu.lib().moty_cuda_set_moe_fast_path(0)
        slow = m.d1(x, logits)
        gpu.lib().moty_cuda_set_moe_fast_path(prev)
        assert same_bits(fast, slow) and same_bits(fast2, slow) and same_bits(split, slow)
        assert same_bits(coop, slow) and same_bits(coop2, slow)
    if small and (lo, hi) == (0, E):
        cat = lambda k, j: np.concatenate([p[j] for p in packs[k]])
        ex = Experts(E, K, I, D, cat("g", 0), cat("u", 0), cat("d", 0), cat("g", 1), cat("u", 1), cat("d", 1))
        assert same_bits(fast, oracle.moe_q4r4(ex, x, logits)[0])


@pytest.mark.parametrize("E,K,I,D,S,lo,hi", [(8, 2, 256, 256, 300, 0, 8), (64, 8, 1024, 2048, 512, 0, 64), (4, 2, 384, 512, 700, 0, 4),
                                             (16, 4, 144, 272, 40, 0, 16), (16, 4, 256, 384, 100, 4, 12), (8, 8, 128, 128, 33, 0, 8)])
def test_moe_q8_batch_on_tensor_cores(gpu, oracle, E, K, I, D, S, lo, hi):
    """Batches whose experts see 8+ routed rows each run the grouped products on tcgen05 (gate + up + SiLU in one pass,
    work list from the routing plan).  Same bits as the mma.sync tile path and as the CPU reference: 16- to 128-row
    tiles, FFN widths and hidden sizes off the 128-row / 128-byte blocks, the OLMoE layer shape at its 512-token
    prompt, an expert shard (rows of non-resident experts contribute nothing), twice in a row on other inputs."""
    from oracle import Experts
    rng = np.random.default_rng(E * 1000 + S + lo)
    g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
    d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
    gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
    ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
    m = gpu.Moe(E, K, I, D, e_lo=lo, e_hi=hi)
    for e in range(lo, hi):
        m.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
    L = gpu.lib()
    for trial in range(2):
        x = rng.standard_normal((S, D)).astype(np.float32)
        logits = (rng.standard_normal((S, E)) * 0.5).astype(np.float32)
        prev = L.moty_cuda_set_moe_batch_path(1)
        tc = m.batch(x, logits); tc_ol = m.olmoe(x, logits, 1)
        L.moty_cuda_set_moe_batch_path(0)
        tiles = m.batch(x, logits); tiles_ol = m.olmoe(x, logits, 1)
        L.moty_cuda_set_moe_batch_path(prev)
        assert same_bits(tc, tiles) and same_bits(tc_ol, tiles_ol)
        assert L.moty_cuda_kernel_status(0, None) == 0
    if (lo, hi) == (0, E):
        assert same_bits(tc, oracle.moe_batch(Experts(E, K, I, D, g, u, d, gs, us, ds), x, logits)[0])


def test_moe_int4_experts_golden(gpu):
    """LFM2's int4 experts (ebits = 4: per-row nibble rows, nn/moe.c:42,99-103,138,193-198) uploaded through
    moty_cuda_moe_upload_expert_i4: vectors from the compiled reference's blocks over the PACKED rows, decode and batch,
    softmax and sigmoid + bias gates, bit for bit (router on the GPU as an int8 matrix, and with logits handed in)."""
    g = golden("blocks_i4")
    E, K, I, D = (int(v) for v in g["dims"])
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert_i4(e, g["g4"][e], g["gs"][e], g["u4"][e], g["us"][e], g["d4"][e], g["ds"][e])
    for router in (None, gpu.Mat.i8(g["rq"], g["rs"])):
        m.set_router(router)
        lg = (lambda S: g[f"logits{S}"]) if router is None else (lambda S: None)
        m.set_sigmoid_gate(False)
        assert same_bits(m.d1(g["x1"], lg(1)), g["out_topk1"]) and same_bits(m.batch(g["x7"], lg(7)), g["out_topk7"])
        m.set_sigmoid_gate(True, g["bias"])
        assert same_bits(m.d1(g["x1"], lg(1)), g["out_sig1"]) and same_bits(m.batch(g["x7"], lg(7)), g["out_sig7"])
    q = gpu.Moe(E, K, I, D, efmt=gpu.WF_Q4R4)
    with pytest.raises(gpu.MotyCudaError, match="MOTY_WF_I8"):
        q.upload_expert_i4(0, g["g4"][0], g["gs"][0], g["u4"][0], g["us"][0], g["d4"][0], g["ds"][0])


def test_moe_sigmoid_gate_golden_and_oracle(gpu, oracle):
    """LFM2's gate (sigmoid + expert bias, nn/moe.c:10-25) around int8 experts: vectors from the compiled reference's
    moty_nn_moe_sigmoid_d1 / _batch bit for bit (router on the GPU as an int8 matrix, and with logits handed in), then
    random layers against the oracle on every batch path (decode, mma.sync tiles, tensor cores)."""
    from oracle import Experts
    g = golden("blocks_sigmoid")
    E, K, I, D = (int(v) for v in g["dims"])
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert(e, g["g"][e], g["gs"][e], g["u"][e], g["us"][e], g["d"][e], g["ds"][e])
    for bias, tag in ((g["bias"], "bias"), (None, "nobias")):
        m.set_sigmoid_gate(True, bias)
        m.set_router(None)
        assert same_bits(m.d1(g["x1"], g["logits1"]), g[f"out_{tag}1"])
        assert same_bits(m.batch(g["x9"], g["logits9"]), g[f"out_{tag}9"])
        m.set_router(gpu.Mat.i8(g["rq"], g["rs"]))
        assert same_bits(m.d1(g["x1"]), g[f"out_{tag}1"]) and same_bits(m.batch(g["x9"]), g[f"out_{tag}9"])
    m.set_sigmoid_gate(False)                                   # back to softmax: another result
    m.set_router(None)
    assert not same_bits(m.d1(g["x1"], g["logits1"]), g["out_bias1"])
    rng = np.random.default_rng(77)
    E, K, I, D = 32, 4, 256, 512                                # the LFM2-8B-A1B gate: 32 experts, top-4
    gq = rng.integers(-127, 128, (E, I, D), dtype=np.int8); uq = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
    dq = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
    gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
    ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
    ex = Experts(E, K, I, D, gq, uq, dq, gs, us, ds)
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert(e, gq[e], gs[e], uq[e], us[e], dq[e], ds[e])
    bias = (rng.standard_normal(E) * 0.2).astype(np.float32)
    m.set_sigmoid_gate(True, bias)
    for S in (1, 7, 200):                                       # decode, mma.sync tiles, tensor cores (25 rows per expert)
        x = rng.standard_normal((S, D)).astype(np.float32); lg = rng.standard_normal((S, E)).astype(np.float32)
        got = m.d1(x, lg) if S == 1 else m.batch(x, lg)
        assert same_bits(got, oracle.moe_sigmoid(ex, x, lg, bias)[0]), S


def test_gemma_attention_golden_and_oracle(gpu, oracle):
    """gemma's attention core (engines/gemma.c:299-386): (1 + w) norms, value norm, p-RoPE on pairs (j, j + hd/2), the
    sliding window, a given score scale.  Against the vectors composed from the engine's own static functions, then at
    the Gemma-4-12B head shape (16 query / 8 KV heads of 256, window 1024) against the oracle: a prompt that crosses the
    window, decode steps past it, and a global layer with partial rotation."""
    from oracle import AttnCache
    from test_oracle import _gemma_attn_cases
    g = golden("attn_gemma")
    one = np.float32(1)
    for tag, cf in _gemma_attn_cases().items():
        get = lambda nm: (one + g[f"{nm}_{tag}"]).astype(np.float32) if f"{nm}_{tag}" in g else None
        a = gpu.Attn(cf["H"], cf["KV"], cf["hd"], 16, theta=1e4, eps=1e-6, rot=cf["rot"], qn=get("qn"), kn=get("kn"), vn=get("vn"),
                     kv8=cf["kv8"], gemma=True, window=cf["window"], scale=cf["scale"])
        pos = 0
        for step, S in enumerate((5, 1, 3, 4)):
            want = g[f"ctx_{tag}_{step}"]
            y = a.core(g[f"q_{tag}_{step}"], g[f"k_{tag}_{step}"], g[f"v_{tag}_{step}"], pos)
            tol = 2e-3 if cf["kv8"] else 5e-5
            assert np.abs(y - want).max() <= tol * np.abs(want).max(), (tag, step, float(np.abs(y - want).max()))
            pos += S
        a.close()
    rng = np.random.default_rng(12)
    H, KV, hd, max_t = 16, 8, 256, 1400
    for window, rot, kv8 in ((1024, 128, False), (0, 32, False), (1024, 128, True)):
        w = lambda: (rng.standard_normal(hd) * 0.1).astype(np.float32)
        qn, kn, vn = w(), w(), w()
        cache = AttnCache(H, KV, hd, max_t, theta=1e4, eps=1e-6, rot=rot, qn=qn, kn=kn, vn=vn, kv8=kv8, gemma=True, window=window, scale=0.0)
        a = gpu.Attn(H, KV, hd, max_t, theta=1e4, eps=1e-6, rot=rot, qn=one + qn, kn=one + kn, vn=one + vn, kv8=kv8, gemma=True, window=window)
        pos = 0
        for S in (900, 300, 1, 1, 9):                           # the second prompt chunk crosses the window; decode steps past it
            q = rng.standard_normal((S, H * hd)).astype(np.float32)
            k = rng.standard_normal((S, KV * hd)).astype(np.float32); v = rng.standard_normal((S, KV * hd)).astype(np.float32)
            yo = oracle.attn_core(q.copy(), k.copy(), v.copy(), pos, cache)
            y = a.core(q, k, v, pos)
            tol = 2e-3 if kv8 else 5e-5
            err, mag = float(np.abs(y - yo).max()), float(np.abs(yo).max())
            assert err <= tol * mag, (window, rot, kv8, S, pos, err, mag)
            pos += S
        a.close()
