"""Generate tests/golden/*.npz from the UNMODIFIED reference.

Run where the reference checkout exists (it is compiled by oracle/Makefile into
oracle/_ref and called through ctypes):

    python tests/golden/make_golden.py

Every fixture stores the seeded inputs together with the outputs the
reference's own compiled code produced for them, so the tests need neither the
reference sources nor its build.  Input recipes mirror the reference's unit
tests: full-range int8 weights including -128 with activations in [-127, 127]
(tests/simd_tests.c:22-44), ragged output counts and token counts 1/5/7/37
(tests/q4r4_tests.c:176-212), random (E, K) routing rows (tests/moe_tests.c:15-39).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import Experts, Ref, WF_I8, WF_Q4R4, build  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def main():
    build()
    r = Ref()
    rng = np.random.default_rng(20240607)
    save = lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw)

    # ---- f16 conversions: every half code, and floats around every rounding case
    codes = np.arange(65536, dtype=np.uint32)
    f = np.array([r.f16_to_f32(int(h)) for h in codes], np.float32)
    probe = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5, -6.1e-5, 1e9, -1e9], np.float32),
        (f[np.isfinite(f)][::97] * np.float32(1.0004883)).astype(np.float32),
    ])
    h = np.array([r.f32_to_f16(v) for v in probe], np.uint16)
    save("f16", f16_to_f32_bits=f.view(np.uint32), probe=probe, probe_f16=h)

    # ---- dot_i8i8 / dot_i4i8: exact int32
    ns = [1, 2, 3, 4, 5, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 1000, 4096]
    dots = {}
    for n in ns:
        w = rng.integers(-128, 128, n, dtype=np.int8)
        x = rng.integers(-127, 128, n, dtype=np.int8)
        w4 = rng.integers(0, 256, (n + 1) // 2, dtype=np.uint8)
        dots[f"w{n}"] = w; dots[f"x{n}"] = x; dots[f"w4_{n}"] = w4
        dots[f"d{n}"] = np.int32(r.dot_i8i8(w, x)); dots[f"d4_{n}"] = np.int32(r.dot_i4i8(w4, x))
    # worst case magnitudes
    w = np.full(16384, -128, np.int8); x = np.full(16384, -127, np.int8)
    dots["wmax"] = w; dots["xmax"] = x; dots["dmax"] = np.int32(r.dot_i8i8(w, x))
    save("dots", ns=np.array(ns), **dots)

    # ---- activation quantizers
    q = {}
    for n in (1, 7, 32, 100, 1000, 1024, 3072):
        x = (rng.standard_normal(n) * rng.choice([1e-3, 1.0, 50.0])).astype(np.float32)
        qq, s = r.qrow_i8(x)
        q[f"x{n}"] = x; q[f"q{n}"] = qq; q[f"s{n}"] = np.float32(s)
    x0 = np.zeros(64, np.float32)                     # all-zero row: the scale floor
    qq, s = r.qrow_i8(x0); q["xzero"] = x0; q["qzero"] = qq; q["szero"] = np.float32(s)
    xt = np.array([0.5, 1.5, 2.5, -0.5, -1.5, 127.0, -127.0, 63.5], np.float32)   # ties: round half to even
    qq, s = r.qrow_i8(xt); q["xties"] = xt; q["qties"] = qq; q["sties"] = np.float32(s)
    xg = rng.standard_normal((5, 256)).astype(np.float32); xg[1, 32:64] = 0; xg[2] *= 1e-20
    a, b, c = r.quant_g32(xg)
    save("quant", ns=np.array([1, 7, 32, 100, 1000, 1024, 3072]), g32_x=xg, g32_q=a, g32_s=b, g32_sum=c, **q)

    # ---- weight quantizers + drivers
    for tag, (O, I) in {"a": (37, 96), "b": (64, 1024), "c": (130, 256)}.items():
        Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
        Wf[0, :32] = 0                                    # an all-zero group
        q8, s8 = r.quantize_rows(Wf)
        q4, s16 = r.pack_q4r4(Wf)
        qi4, si4 = r.pack_int4(Wf)
        W8 = rng.integers(-127, 128, (O, I), dtype=np.int8)
        sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
        d = dict(Wf=Wf, q8=q8, s8=s8, q4=q4, s16=s16, qi4=qi4, si4=si4, W8=W8, sc=sc)
        for S in (1, 2, 3, 4, 5, 7, 16, 37):
            x = rng.standard_normal((S, I)).astype(np.float32)
            d[f"x{S}"] = x
            d[f"y8_{S}"] = r.matmul_q_s(x, W8, sc)
            d[f"y4_{S}"] = r.matmul_q4r4_s(x, q4, s16, O)
        save("matmul_" + tag, O=np.int32(O), I=np.int32(I), **d)

    # ---- router
    rt = {}
    for tag, (E, K, sd) in {"a": (128, 8, 0.05), "b": (64, 8, 1.0), "c": (16, 2, 3.0), "d": (7, 7, 0.5)}.items():
        lg = (rng.standard_normal((48, E)) * sd).astype(np.float32)
        lg[0, :] = 0.25                                   # all equal: ties go to the lowest indices
        idx, w, probs = r.route_topk(lg, K)
        idx0, w0 = r.moe_topk(probs, K, 0)
        rt.update({f"lg_{tag}": lg, f"idx_{tag}": idx, f"w_{tag}": w, f"p_{tag}": probs, f"idx0_{tag}": idx0, f"w0_{tag}": w0,
                   f"K_{tag}": np.int32(K)})
    v = rng.standard_normal(151936).astype(np.float32); v[77] = v.max(); v[9000] = v.max()
    rt["argmax_v"] = v[:5000].copy(); rt["argmax_i"] = np.int32(r.argmax(v[:5000]))
    save("router", **rt)

    # ---- blocks: FFN and MoE
    D, I = 128, 256
    blk = {}
    Wg, Wu, Wd = ((rng.standard_normal(s) * 0.05).astype(np.float32) for s in ((I, D), (I, D), (D, I)))
    G, U, Dn = r.quantize_rows(Wg), r.quantize_rows(Wu), r.quantize_rows(Wd)
    G4, U4, D4 = r.pack_q4r4(Wg), r.pack_q4r4(Wu), r.pack_q4r4(Wd)
    blk.update(gq=G[0], gs=G[1], uq=U[0], us=U[1], dq=Dn[0], ds=Dn[1],
               g4=G4[0], g4s=G4[1], u4=U4[0], u4s=U4[1], d4=D4[0], d4s=D4[1])
    for S in (1, 5):
        x = rng.standard_normal((S, D)).astype(np.float32)
        blk[f"ffn_x{S}"] = x
        blk[f"ffn8_{S}"] = r.dense_ffn(WF_I8, x, I, G[0], G[1], U[0], U[1], Dn[0], Dn[1])
        blk[f"ffn4_{S}"] = r.dense_ffn(WF_Q4R4, x, I, G4[0], G4[1], U4[0], U4[1], D4[0], D4[1])
    E, K, I2, D2 = 8, 2, 64, 128
    g = rng.integers(-127, 128, (E, I2, D2), dtype=np.int8); u = rng.integers(-127, 128, (E, I2, D2), dtype=np.int8)
    d = rng.integers(-127, 128, (E, D2, I2), dtype=np.int8)
    gs = rng.uniform(0.001, 0.02, (E, I2)).astype(np.float32); us = rng.uniform(0.001, 0.02, (E, I2)).astype(np.float32)
    ds = rng.uniform(0.001, 0.02, (E, D2)).astype(np.float32)
    ex = Experts(E, K, I2, D2, g, u, d, gs, us, ds)
    router = (rng.standard_normal((E, D2)) * 0.1).astype(np.float32)
    rq, rs = r.quantize_rows(router)
    blk.update(moe_g=g, moe_u=u, moe_d=d, moe_gs=gs, moe_us=us, moe_ds=ds, moe_rq=rq, moe_rs=rs,
               moe_dims=np.array([E, K, I2, D2], np.int32))
    for S in (1, 9):
        x = rng.standard_normal((S, D2)).astype(np.float32)
        logits = r.matmul_q_s(x, rq, rs)
        blk[f"moe_x{S}"] = x; blk[f"moe_logits{S}"] = logits
        blk[f"moe_out{S}"] = r.moe_topk_block(ex, x, router_q=rq, router_qs=rs)
        o, idx, w = r.olmoe_moe(ex, x, logits, 0)
        blk[f"olmoe_out{S}"] = o; blk[f"olmoe_idx{S}"] = idx; blk[f"olmoe_w{S}"] = w
    save("blocks", **blk)

    # ---- Q8R4, the int8 sibling of Q4R4 (its own random stream: added after the files above were fixed)
    rq8 = np.random.default_rng(20260811)
    d = {}
    for tag, (O, I) in {"a": (37, 96), "b": (66, 512)}.items():
        Wf = (rq8.standard_normal((O, I)) * 0.02).astype(np.float32)
        Wf[0, :32] = 0                                    # an all-zero group: scale 0, codes 0
        q8, s16 = r.pack_q8r4(Wf)
        d.update({f"Wf_{tag}": Wf, f"q8_{tag}": q8, f"s16_{tag}": s16, f"O_{tag}": np.int32(O)})
        for S in (1, 3, 4, 5, 16, 37):
            x = rq8.standard_normal((S, I)).astype(np.float32)
            d[f"x_{tag}_{S}"] = x
            d[f"y_{tag}_{S}"] = r.matmul_q8r4_s(x, q8, s16, O)
    save("matmul_q8r4", **d)

    # ---- WF_I4G, grouped int4 (group 32), integer path (IDOT4=1): needs the reference's AVX512-VNNI tier
    if r.has_i4g_idot():
        rg = np.random.default_rng(20260812)
        d = {}
        for tag, (O, I) in {"a": (37, 128), "b": (40, 1792)}.items():
            Wf = (rg.standard_normal((O, I)) * 0.02).astype(np.float32)
            Wf[0, :32] = 0                                # an all-zero group: floor scale, codes 8
            q4, sc = r.pack_int4_grouped(Wf)
            d.update({f"q4_{tag}": q4, f"scale_{tag}": sc})
            if tag == "a":
                d["Wf_a"] = Wf                            # pins the packer too
            for S in (1, 2, 5, 9):
                x = rg.standard_normal((S, I)).astype(np.float32)
                d[f"x_{tag}_{S}"] = x
                d[f"y_{tag}_{S}"] = r.matmul_i4g_idot_s(x, q4, sc)
        save("matmul_i4g", **d)
    else:
        print("WF_I4G vectors not regenerated: the reference build here has no AVX512-VNNI tier")

    # ---- attention core between the projections (nn/attn.c:29-74), composed from the reference's own functions
    from oracle import AttnCache
    ra = np.random.default_rng(20260813)
    d = {}
    cases = {"a": dict(H=4, KV=2, hd=64, rot=64, norm=True, kv8=False), "b": dict(H=8, KV=2, hd=128, rot=64, norm=False, kv8=False),
             "c": dict(H=4, KV=2, hd=64, rot=64, norm=True, kv8=True), "d": dict(H=6, KV=3, hd=96, rot=32, norm=True, kv8=True)}
    for tag, cf in cases.items():
        hd = cf["hd"]
        qn = ra.uniform(0.5, 1.5, hd).astype(np.float32) if cf["norm"] else None
        kn = ra.uniform(0.5, 1.5, hd).astype(np.float32) if cf["norm"] else None
        cache = AttnCache(cf["H"], cf["KV"], hd, 16, theta=1e6, eps=1e-6, rot=cf["rot"], qn=qn, kn=kn, kv8=cf["kv8"])
        d[f"cfg_{tag}"] = np.array([cf["H"], cf["KV"], hd, cf["rot"], int(cf["norm"]), int(cf["kv8"])], np.int32)
        if cf["norm"]:
            d[f"qn_{tag}"] = qn; d[f"kn_{tag}"] = kn
        pos = 0
        for step, S in enumerate((5, 1, 3)):
            q = ra.standard_normal((S, cf["H"] * hd)).astype(np.float32)
            k = ra.standard_normal((S, cf["KV"] * hd)).astype(np.float32)
            v = ra.standard_normal((S, cf["KV"] * hd)).astype(np.float32)
            d[f"q_{tag}_{step}"] = q; d[f"k_{tag}_{step}"] = k; d[f"v_{tag}_{step}"] = v
            d[f"ctx_{tag}_{step}"] = r.attn_core(q.copy(), k.copy(), v.copy(), pos, cache)
            pos += S
    save("attn", **d)
    sigmoid_blocks(r, save)
    gelu_vectors(r, save)
    gemma_attn_vectors(r, save)
    print("golden vectors written to", OUT, "by reference tier", r.tier)


def sigmoid_blocks(r, save):
    """The MoE block behind LFM2's sigmoid + expert-bias gate (moty_nn_moe_sigmoid_d1 / _batch, nn/moe.c:10-25,154,207),
    int8 experts and an int8 router; its own random stream (added after the files above were fixed).  `only` lets this
    one file be written without touching the others:  python tests/golden/make_golden.py sigmoid"""
    rs_ = np.random.default_rng(20261125)
    E, K, I2, D2 = 16, 4, 64, 128
    g = rs_.integers(-127, 128, (E, I2, D2), dtype=np.int8); u = rs_.integers(-127, 128, (E, I2, D2), dtype=np.int8)
    d = rs_.integers(-127, 128, (E, D2, I2), dtype=np.int8)
    gs = rs_.uniform(0.001, 0.02, (E, I2)).astype(np.float32); us = rs_.uniform(0.001, 0.02, (E, I2)).astype(np.float32)
    ds = rs_.uniform(0.001, 0.02, (E, D2)).astype(np.float32)
    ex = Experts(E, K, I2, D2, g, u, d, gs, us, ds)
    rq, rsc = r.quantize_rows((rs_.standard_normal((E, D2)) * 0.1).astype(np.float32))
    bias = (rs_.standard_normal(E) * 0.3).astype(np.float32)
    blk = dict(g=g, u=u, d=d, gs=gs, us=us, ds=ds, rq=rq, rs=rsc, bias=bias, dims=np.array([E, K, I2, D2], np.int32))
    for S in (1, 9):
        x = rs_.standard_normal((S, D2)).astype(np.float32)
        blk[f"x{S}"] = x; blk[f"logits{S}"] = r.matmul_q_s(x, rq, rsc)
        blk[f"out_bias{S}"] = r.moe_sigmoid_block(ex, x, bias, rq, rsc)
        blk[f"out_nobias{S}"] = r.moe_sigmoid_block(ex, x, None, rq, rsc)
    save("blocks_sigmoid", **blk)


def i4_expert_blocks(r, save):
    """The MoE block over per-row int4 experts (LFM2's ebits = 4; nn/moe.c:42,99-103,138,193-198), both gates, decode and
    batch (the batch path through moty_matmul_i4_s with IDOT4=1); its own file and random stream:
    python tests/golden/make_golden.py i4experts"""
    rs_ = np.random.default_rng(20261128)
    E, K, I2, D2 = 12, 3, 96, 192                       # row lengths that leave a scalar tail behind the 64-wide steps
    g4 = rs_.integers(0, 256, (E, I2, D2 // 2), dtype=np.uint8); u4 = rs_.integers(0, 256, (E, I2, D2 // 2), dtype=np.uint8)
    d4 = rs_.integers(0, 256, (E, D2, I2 // 2), dtype=np.uint8)
    gs = rs_.uniform(0.01, 0.2, (E, I2)).astype(np.float32); us = rs_.uniform(0.01, 0.2, (E, I2)).astype(np.float32)
    ds = rs_.uniform(0.01, 0.2, (E, D2)).astype(np.float32)
    ex4 = Experts(E, K, I2, D2, g4, u4, d4, gs, us, ds)
    rq, rsc = r.quantize_rows((rs_.standard_normal((E, D2)) * 0.1).astype(np.float32))
    bias = (rs_.standard_normal(E) * 0.3).astype(np.float32)
    blk = dict(g4=g4, u4=u4, d4=d4, gs=gs, us=us, ds=ds, rq=rq, rs=rsc, bias=bias, dims=np.array([E, K, I2, D2], np.int32))
    for S in (1, 7):
        x = rs_.standard_normal((S, D2)).astype(np.float32)
        blk[f"x{S}"] = x; blk[f"logits{S}"] = r.matmul_q_s(x, rq, rsc)
        blk[f"out_topk{S}"] = r.moe_i4_block(ex4, x, rq, rsc)
        blk[f"out_sig{S}"] = r.moe_i4_block(ex4, x, rq, rsc, sig=True, bias=bias)
    save("blocks_i4", **blk)


def i4g_f32_vectors(r, save):
    """WF_I4G through the reference's default product, f32 x dequantized int4 (i4g_f32_rows, nn/matmul.c:196-253).  The
    driver latches IDOT4 on its first call, so this function must run in a process started with IDOT4=0 (the __main__
    branch below re-executes itself that way); the row length 96 takes this product under either setting.
    python tests/golden/make_golden.py i4g_f32"""
    assert os.environ.get("IDOT4") == "0"
    rg = np.random.default_rng(20261129)
    d = {}
    for tag, (O, I, S) in {"a": (40, 256, 3), "b": (17, 96, 2), "c": (64, 1024, 1)}.items():
        q4 = rg.integers(0, 256, (O, I // 2), dtype=np.uint8)
        sc = rg.uniform(0.001, 0.02, (O, I // 32)).astype(np.float32)
        x = rg.standard_normal((S, I)).astype(np.float32)
        d[f"q4_{tag}"] = q4; d[f"s_{tag}"] = sc; d[f"x_{tag}"] = x; d[f"y_{tag}"] = r.matmul_i4g_any(x, q4, sc)
    save("i4g_f32", **d)


def gelu_vectors(r, save):
    """gemma's GeGLU element step from the engine's own static gelu_tanh (engines/gemma.c:389-391,398): a dense sweep
    of the activation's working range, large and tiny magnitudes, and normal draws; its own file and random stream."""
    rg = np.random.default_rng(20261126)
    g = np.concatenate([np.linspace(-12, 12, 6001, dtype=np.float32), rg.standard_normal(6000).astype(np.float32) * 3,
                        (rg.standard_normal(500) * 1e-4).astype(np.float32), np.array([0.0, -0.0, 30.0, -30.0, 1e-20, 88.0, -88.0], np.float32)])
    u = rg.standard_normal(g.size).astype(np.float32)
    save("gelu", g=g, u=u, out=r.gelu_mul(g, u))


GEMMA_ATTN_CASES = {
    "s": dict(H=4, KV=2, hd=64, rot=32, window=6, scale=0.0, norm=True, vnorm=True, kv8=False),      # sliding: full p-RoPE (hd/2 pairs)
    "t": dict(H=4, KV=2, hd=64, rot=32, window=5, scale=0.0, norm=True, vnorm=False, kv8=True),      # sliding, int8 cache
    "g": dict(H=6, KV=2, hd=128, rot=16, window=0, scale=0.0625, norm=True, vnorm=True, kv8=False),  # global: partial rotation, given scale
}


def gemma_attn_vectors(r, save):
    """gemma's attention core (engines/gemma.c:299-386 without projections, shared-KV layers and k_eq_v), composed from
    the engine's own static gnorm_row / gemma_rope_head and the reference's score / softmax / accumulate functions with
    the sliding window's start; four calls per case on one cache (5, 1, 3, 4 tokens: past the window)."""
    from oracle import AttnCache
    ra = np.random.default_rng(20261127)
    d = {}
    for tag, cf in GEMMA_ATTN_CASES.items():
        hd = cf["hd"]
        w = lambda: (ra.standard_normal(hd) * 0.2).astype(np.float32)
        qn, kn = (w(), w()) if cf["norm"] else (None, None)
        vn = w() if cf["vnorm"] else None
        cache = AttnCache(cf["H"], cf["KV"], hd, 16, theta=1e4, eps=1e-6, rot=cf["rot"], qn=qn, kn=kn, kv8=cf["kv8"],
                          gemma=True, window=cf["window"], scale=cf["scale"], vn=vn)
        for nm, arr in (("qn", qn), ("kn", kn), ("vn", vn)):
            if arr is not None:
                d[f"{nm}_{tag}"] = arr
        pos = 0
        for step, S in enumerate((5, 1, 3, 4)):
            q = ra.standard_normal((S, cf["H"] * hd)).astype(np.float32)
            k = ra.standard_normal((S, cf["KV"] * hd)).astype(np.float32)
            v = ra.standard_normal((S, cf["KV"] * hd)).astype(np.float32)
            d[f"q_{tag}_{step}"] = q; d[f"k_{tag}_{step}"] = k; d[f"v_{tag}_{step}"] = v
            d[f"ctx_{tag}_{step}"] = r.attn_core(q.copy(), k.copy(), v.copy(), pos, cache)
            pos += S
    save("attn_gemma", **d)


if __name__ == "__main__":
    if sys.argv[1:] == ["gemma_attn"]:
        build()
        gemma_attn_vectors(Ref(), lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw))
    elif sys.argv[1:] == ["gelu"]:
        build()
        gelu_vectors(Ref(), lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw))
    elif sys.argv[1:] == ["i4g_f32"]:
        if os.environ.get("IDOT4") != "0":                  # the reference reads IDOT4 once per process
            import subprocess
            sys.exit(subprocess.call([sys.executable, os.path.abspath(__file__), "i4g_f32"], env={**os.environ, "IDOT4": "0"}))
        build()
        i4g_f32_vectors(Ref(), lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw))
    elif sys.argv[1:] == ["i4experts"]:
        build()
        i4_expert_blocks(Ref(), lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw))
    elif sys.argv[1:] == ["sigmoid"]:
        build()
        sigmoid_blocks(Ref(), lambda name, **kw: np.savez_compressed(os.path.join(OUT, name + ".npz"), **kw))
    else:
        main()
