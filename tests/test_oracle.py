"""CPU: the C restatement against the golden vectors (made by the reference's own
compiled code) and, where the reference library exists, bit for bit against it."""
import os

import numpy as np
import pytest

from conftest import golden, same_bits


def test_f16_tables(oracle):
    g = golden("f16")
    got = np.array([oracle.f16_to_f32(h) for h in range(65536)], np.float32).view(np.uint32)
    assert same_bits(got, g["f16_to_f32_bits"])
    h = np.array([oracle.f32_to_f16(v) for v in g["probe"]], np.uint16)
    assert same_bits(h, g["probe_f16"])


def test_dots_exact(oracle):
    g = golden("dots")
    for n in g["ns"]:
        assert oracle.dot_i8i8(g[f"w{n}"], g[f"x{n}"]) == int(g[f"d{n}"])
        assert oracle.dot_i4i8(g[f"w4_{n}"], g[f"x{n}"]) == int(g[f"d4_{n}"])
    assert oracle.dot_i8i8(g["wmax"], g["xmax"]) == int(g["dmax"]) == 128 * 127 * 16384


def test_quantizers(oracle):
    g = golden("quant")
    for n in list(g["ns"]) + ["zero", "ties"]:
        q, s = oracle.qrow_i8(g[f"x{n}"])
        assert same_bits(q, g[f"q{n}"]) and np.float32(s) == g[f"s{n}"]
    xq, xs, xsum = oracle.quant_g32(g["g32_x"])
    assert same_bits(xq, g["g32_q"]) and same_bits(xs, g["g32_s"]) and same_bits(xsum, g["g32_sum"])
    # reconstruction bound of the reference's own test (tests/simd_tests.c:127-145)
    x = g["x1024"]; q, s = oracle.qrow_i8(x)
    assert np.all(np.abs(x - s * q.astype(np.float32)) <= s / 2 * 1.0001)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_drivers(oracle, tag):
    g = golden("matmul_" + tag)
    O, I = int(g["O"]), int(g["I"])
    q8, s8 = oracle.quantize_rows(g["Wf"])
    assert same_bits(q8, g["q8"]) and same_bits(s8, g["s8"])
    q4, s16 = oracle.pack_q4r4(g["Wf"])
    assert same_bits(q4, g["q4"]) and same_bits(s16, g["s16"])
    qi4, si4 = oracle.pack_int4(g["Wf"])
    assert same_bits(qi4, g["qi4"]) and same_bits(si4, g["si4"])
    for S in (1, 2, 3, 4, 5, 7, 16, 37):
        x = g[f"x{S}"]
        y, acc = oracle.matmul_q_s(x, g["W8"], g["sc"], want_acc=True)
        assert same_bits(y, g[f"y8_{S}"])
        xi, sx = oracle.qrows_i8(x)
        assert np.array_equal(acc, xi.astype(np.int32) @ g["W8"].astype(np.int32).T)
        assert same_bits(oracle.matmul_q4r4_s(x, g["q4"], g["s16"], O), g[f"y4_{S}"])


def test_q8r4_drivers(oracle):
    """Q8R4 packer and product against vectors from the reference build (nn/quant.c:135-155,
    nn/matmul.c:435-461)."""
    g = golden("matmul_q8r4")
    for tag in ("a", "b"):
        O = int(g[f"O_{tag}"])
        q8, s16 = oracle.pack_q8r4(g[f"Wf_{tag}"])
        assert same_bits(q8, g[f"q8_{tag}"]) and same_bits(s16, g[f"s16_{tag}"])
        for S in (1, 3, 4, 5, 16, 37):
            assert same_bits(oracle.matmul_q8r4_s(g[f"x_{tag}_{S}"], q8, s16, O), g[f"y_{tag}_{S}"])


def test_i4g_drivers(oracle):
    """WF_I4G (grouped int4, group 32): packer and the integer path of the product against vectors from the
    reference's AVX512-VNNI build (nn/quant.c:57-83, nn/matmul.c:164-197 with IDOT4=1)."""
    g = golden("matmul_i4g")
    q4, sc = oracle.pack_int4_grouped(g["Wf_a"])
    assert same_bits(q4, g["q4_a"]) and same_bits(sc, g["scale_a"])
    for tag in ("a", "b"):
        for S in (1, 2, 5, 9):
            assert same_bits(oracle.matmul_i4g_idot_s(g[f"x_{tag}_{S}"], g[f"q4_{tag}"], g[f"scale_{tag}"]), g[f"y_{tag}_{S}"])


def _attn_golden_cases():
    from oracle import AttnCache
    g = golden("attn")
    for tag in ("a", "b", "c", "d"):
        H, KV, hd, rot, norm, kv8 = (int(v) for v in g[f"cfg_{tag}"])
        qn = g[f"qn_{tag}"] if norm else None; kn = g[f"kn_{tag}"] if norm else None
        mk = lambda: AttnCache(H, KV, hd, 16, theta=1e6, eps=1e-6, rot=rot, qn=qn, kn=kn, kv8=bool(kv8))
        steps = [(g[f"q_{tag}_{i}"], g[f"k_{tag}_{i}"], g[f"v_{tag}_{i}"], g[f"ctx_{tag}_{i}"]) for i in range(3)]
        yield tag, mk, steps


def test_attn_core_golden(oracle):
    """The attention core (nn/attn.c:29-74: QK-norm, RoPE, f32 and int8 KV store, scores, softmax, accumulation)
    against vectors composed from the reference's own functions.  The reference's tiers sum in different orders
    and contract multiply-adds, so this level is pinned by tolerance: 5e-6 of the output magnitude."""
    for tag, mk, steps in _attn_golden_cases():
        cache = mk(); pos = 0
        for q, k, v, ctx in steps:
            y = oracle.attn_core(q.copy(), k.copy(), v.copy(), pos, cache)
            assert np.abs(y - ctx).max() <= 5e-6 * np.abs(ctx).max(), tag
            pos += q.shape[0]


def test_q4r4_batch_is_not_row_invariant(oracle):
    """The reference folds the -8 offset differently for tokens inside a complete
    group of 4 (nn/matmul.c:397-402): a batch is NOT always bitwise equal to its
    rows run one by one.  The restatement must keep that, so pin it."""
    g = golden("matmul_a")
    O = int(g["O"]); x = g["x5"]
    yb = oracle.matmul_q4r4_s(x, g["q4"], g["s16"], O)
    y1 = np.concatenate([oracle.matmul_q4r4_s(x[i:i + 1], g["q4"], g["s16"], O) for i in range(5)])
    assert same_bits(yb[4], y1[4])                      # the tail token takes the one-token kernel
    np.testing.assert_allclose(yb, y1, rtol=0, atol=1e-5 * np.abs(y1).max())


def test_q8_batch_is_row_invariant(oracle):
    """tests/qwen_tests.c:82-109: an S=4 batch equals four S=1 calls bit for bit."""
    g = golden("matmul_c"); x = g["x4"]
    yb = oracle.matmul_q_s(x, g["W8"], g["sc"])
    y1 = np.concatenate([oracle.matmul_q_s(x[i:i + 1], g["W8"], g["sc"]) for i in range(4)])
    assert same_bits(yb, y1)


def test_router(oracle):
    g = golden("router")
    for tag in "abcd":
        K = int(g[f"K_{tag}"])
        idx, w, probs = oracle.route_topk(g[f"lg_{tag}"], K)
        assert same_bits(idx, g[f"idx_{tag}"]) and same_bits(w, g[f"w_{tag}"]) and same_bits(probs, g[f"p_{tag}"])
        idx0, w0 = oracle.moe_topk(g[f"p_{tag}"], K, 0)
        assert same_bits(idx0, g[f"idx0_{tag}"]) and same_bits(w0, g[f"w0_{tag}"])
        assert list(g[f"idx_{tag}"][0]) == list(range(K))         # all-equal row: lowest indices
    assert oracle.argmax(g["argmax_v"]) == int(g["argmax_i"]) == 77


def test_topk_is_naive_greedy(oracle):
    """tests/moe_tests.c:15-39: identical to a naive greedy pick over random (E, K)."""
    rng = np.random.default_rng(5)
    for _ in range(200):
        E = int(rng.integers(2, 300)); K = int(rng.integers(1, min(E, 16) + 1))
        p = rng.random(E).astype(np.float32)
        idx, w = oracle.moe_topk(p, K, 0)
        order = sorted(range(E), key=lambda e: (-p[e], e))[:K]
        assert list(idx[0]) == order and np.array_equal(w[0], p[order])


def test_blocks(oracle):
    from oracle import Experts
    g = golden("blocks")
    for S in (1, 5):
        x = g[f"ffn_x{S}"]
        assert same_bits(oracle.ffn_q8(x, g["gq"], g["gs"], g["uq"], g["us"], g["dq"], g["ds"]), g[f"ffn8_{S}"])
        assert same_bits(oracle.ffn_q4r4(x, 256, g["g4"], g["g4s"], g["u4"], g["u4s"], g["d4"], g["d4s"]), g[f"ffn4_{S}"])
    E, K, I, D = (int(v) for v in g["moe_dims"])
    ex = Experts(E, K, I, D, g["moe_g"], g["moe_u"], g["moe_d"], g["moe_gs"], g["moe_us"], g["moe_ds"])
    out, _, _ = oracle.moe_d1(ex, g["moe_x1"], g["moe_logits1"])
    assert same_bits(out, g["moe_out1"])
    out, _, _ = oracle.moe_batch(ex, g["moe_x9"], g["moe_logits9"])
    assert same_bits(out, g["moe_out9"])
    for S in (1, 9):
        out, idx, w = oracle.olmoe_moe(ex, g[f"moe_x{S}"], g[f"moe_logits{S}"], 0)
        assert same_bits(out, g[f"olmoe_out{S}"]) and same_bits(idx, g[f"olmoe_idx{S}"]) and same_bits(w, g[f"olmoe_w{S}"])


def test_oracle_equals_reference_build(oracle, ref):
    """Fresh random inputs, both libraries, bit for bit (skipped without the reference)."""
    rng = np.random.default_rng(11)
    for (O, I, S) in ((33, 64, 3), (257, 1024, 9), (64, 3072, 33)):
        W = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
        x = rng.standard_normal((S, I)).astype(np.float32)
        assert same_bits(oracle.matmul_q_s(x, W, sc), ref.matmul_q_s(x, W, sc))
        Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
        a, b = oracle.pack_q4r4(Wf), ref.pack_q4r4(Wf)
        assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])
        assert same_bits(oracle.matmul_q4r4_s(x, a[0], a[1], O), ref.matmul_q4r4_s(x, a[0], a[1], O))
        a, b = oracle.pack_q8r4(Wf), ref.pack_q8r4(Wf)
        assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])
        assert same_bits(oracle.matmul_q8r4_s(x, a[0], a[1], O), ref.matmul_q8r4_s(x, a[0], a[1], O))
    lg = (rng.standard_normal((500, 128)) * 0.05).astype(np.float32)
    Wg = (rng.standard_normal((50, 1024)) * 0.02).astype(np.float32)
    a, b = oracle.pack_int4_grouped(Wg), ref.pack_int4_grouped(Wg)
    assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])
    if ref.has_i4g_idot():                              # the reference takes the integer path only with AVX512-VNNI
        xg = rng.standard_normal((5, 1024)).astype(np.float32)
        assert same_bits(oracle.matmul_i4g_idot_s(xg, a[0], a[1]), ref.matmul_i4g_idot_s(xg, a[0], a[1]))
    a, b = oracle.route_topk(lg, 8), ref.route_topk(lg, 8)
    assert all(same_bits(u, v) for u, v in zip(a, b))


def test_expf_restatement_equals_the_c_library(oracle):
    """SiLU, the router softmax and the output gate of the reference call the C library's expf
    (hw/hw_ops.h:19-26, nn/moe.c:120,197, nn/attn.c:69).  The restatement must give the same bits:
    every 37th float bit pattern over the whole 2^32 range (1.16e8 inputs, all exponents, both signs),
    and EVERY float in [-32, -1/64] and [1/64, 32] -- the range SiLU and softmax arguments live in."""
    assert oracle.expf_mismatches(0, 37, (1 << 32) // 37) == 0
    lo, hi = np.float32(1 / 64).view(np.uint32), np.float32(32).view(np.uint32)
    for sign in (0, 0x80000000):
        assert oracle.expf_mismatches(int(lo) | sign, 1, int(hi) - int(lo) + 1) == 0
    assert oracle.expf(-np.inf) == 0 and oracle.expf(np.inf) == np.inf and np.isnan(oracle.expf(np.nan))


def test_expf_table_is_two_to_the_i_over_32(oracle):
    """Entry i of the restatement's table is 2^(i/32) rounded to nearest f64, less i << 47."""
    mpmath = pytest.importorskip("mpmath")
    mpmath.mp.prec = 200
    for i in range(32):
        d = float(mpmath.power(2, mpmath.mpf(i) / 32))
        bits = int(np.float64(d).view(np.uint64)) - (i << 47)
        assert int(oracle.lib.oracle_exp2_tab_entry(i)) == bits


def test_sigmoid_gate_block_golden(oracle):
    """LFM2's gate (sigmoid + expert bias, nn/moe.c:10-25) around the int8 expert block: the restatement against
    vectors from moty_nn_moe_sigmoid_d1 / _batch of the compiled reference, with and without a bias."""
    from oracle import Experts
    g = golden("blocks_sigmoid")
    E, K, I, D = (int(v) for v in g["dims"])
    ex = Experts(E, K, I, D, g["g"], g["u"], g["d"], g["gs"], g["us"], g["ds"])
    for S in (1, 9):
        assert same_bits(oracle.matmul_q_s(g[f"x{S}"], g["rq"], g["rs"]), g[f"logits{S}"])
        assert same_bits(oracle.moe_sigmoid(ex, g[f"x{S}"], g[f"logits{S}"], g["bias"])[0], g[f"out_bias{S}"])
        assert same_bits(oracle.moe_sigmoid(ex, g[f"x{S}"], g[f"logits{S}"], None)[0], g[f"out_nobias{S}"])
    # the bias moves the selection but not the weights' source: a large bias on one expert forces it in
    b = np.zeros(E, np.float32); b[5] = 10
    _, idx, w = oracle.moe_sigmoid(ex, g["x1"], g["logits1"], b)
    assert idx[0, 0] == 5 and abs(float(w.sum()) - 1) < 1e-6


def test_int4_experts_are_the_int8_blocks_over_unpacked_codes(oracle):
    """LFM2's int4 experts (nn/moe.c:42,99-103,138,193-198): the reference's blocks over the packed nibble rows equal
    the restated int8 blocks over the codes nibble - 8 bit for bit -- decode (dot_i4i8p) and batch (moty_matmul_i4_s with
    IDOT4=1), softmax and sigmoid + bias gates.  That identity is what the GPU upload of such experts relies on."""
    from oracle import Experts, unpack_i4_rows
    g = golden("blocks_i4")
    E, K, I, D = (int(v) for v in g["dims"])
    ex = Experts(E, K, I, D, unpack_i4_rows(g["g4"], D), unpack_i4_rows(g["u4"], D), unpack_i4_rows(g["d4"], I), g["gs"], g["us"], g["ds"])
    assert same_bits(oracle.moe_d1(ex, g["x1"], g["logits1"])[0], g["out_topk1"])
    assert same_bits(oracle.moe_batch(ex, g["x7"], g["logits7"])[0], g["out_topk7"])
    assert same_bits(oracle.moe_sigmoid(ex, g["x1"], g["logits1"], g["bias"])[0], g["out_sig1"])
    assert same_bits(oracle.moe_sigmoid(ex, g["x7"], g["logits7"], g["bias"])[0], g["out_sig7"])


def test_i4g_float_path_golden(oracle):
    """WF_I4G through the reference's default product (f32 x dequantized int4, nn/matmul.c:196-253; vectors generated in
    a process with IDOT4=0): the restatement sums a group in element order, the reference in its SIMD tier's lane order,
    so they agree to the f32 rounding of a 32-term sum (1e-6 of the output magnitude), not bit for bit -- and the vectors
    are NOT the integer path's (which differs by several 1e-3)."""
    g = golden("i4g_f32")
    for t in "abc":
        x, q4, sc, want = g[f"x_{t}"], g[f"q4_{t}"], g[f"s_{t}"], g[f"y_{t}"]
        got = oracle.matmul_i4g_f32_s(x, q4, sc)
        assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max(), t
        if x.shape[1] % 64 == 0:
            assert np.abs(oracle.matmul_i4g_idot_s(x, q4, sc) - want).max() > 1e-4 * np.abs(want).max()


def test_gelu_tanh_golden(oracle):
    """gemma's GeGLU element step: the restatement (with the multiply-add contraction the reference build applies to
    x + 0.044715 x^3) against vectors from the engine's own static gelu_tanh, bit for bit.  Both call the C library's tanhf."""
    g = golden("gelu")
    assert same_bits(oracle.gelu_mul(g["g"], g["u"]), g["out"])


def _gemma_attn_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec); spec.loader.exec_module(mod)
    return mod.GEMMA_ATTN_CASES


def test_gemma_attention_golden(oracle):
    """gemma's attention core -- (1 + w) norms, value norm, p-RoPE on pairs (j, j + hd/2), sliding window, given score
    scale -- against vectors composed from the engine's own static functions and the reference's score / softmax /
    accumulate kernels.  f32 arithmetic in tier-dependent order: 5e-6 of the output magnitude (2e-3 with the int8 cache)."""
    from oracle import AttnCache
    g = golden("attn_gemma")
    for tag, cf in _gemma_attn_cases().items():
        get = lambda nm: g[f"{nm}_{tag}"] if f"{nm}_{tag}" in g else None
        cache = AttnCache(cf["H"], cf["KV"], cf["hd"], 16, theta=1e4, eps=1e-6, rot=cf["rot"], qn=get("qn"), kn=get("kn"),
                          kv8=cf["kv8"], gemma=True, window=cf["window"], scale=cf["scale"], vn=get("vn"))
        pos = 0
        for step, S in enumerate((5, 1, 3, 4)):
            want = g[f"ctx_{tag}_{step}"]
            got = oracle.attn_core(g[f"q_{tag}_{step}"].copy(), g[f"k_{tag}_{step}"].copy(), g[f"v_{tag}_{step}"].copy(), pos, cache)
            tol = 2e-3 if cf["kv8"] else 5e-6
            assert np.abs(got - want).max() <= tol * np.abs(want).max(), (tag, step, float(np.abs(got - want).max()))
            pos += S
