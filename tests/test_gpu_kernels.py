"""GPU parity, kernel level, through the C ABI: bit-exact against the golden
vectors and the CPU oracle."""
import numpy as np
import pytest

from conftest import golden, same_bits

pytestmark = pytest.mark.gpu


def test_dot_i8i8_exact(gpu, oracle):
    g = golden("dots")
    for n in g["ns"]:
        assert int(gpu.dot_i8i8(g[f"w{n}"][None, :], g[f"x{n}"])[0]) == int(g[f"d{n}"])
        assert int(gpu.dot_i4i8(g[f"w4_{n}"], g[f"x{n}"], 1)[0]) == int(g[f"d4_{n}"])
    assert int(gpu.dot_i8i8(g["wmax"][None, :], g["xmax"])[0]) == int(g["dmax"])
    # tests/simd_tests.c:22-44: every n in 1..257 and 4096, weights incl. -128, x in [-127,127]
    rng = np.random.default_rng(1)
    for n in list(range(1, 258)) + [4096]:
        w = rng.integers(-128, 128, (3, n), dtype=np.int8); x = rng.integers(-127, 128, n, dtype=np.int8)
        want = w.astype(np.int64) @ x.astype(np.int64)
        assert np.array_equal(gpu.dot_i8i8(w, x).astype(np.int64), want), n


def test_qrow_i8_bit_exact(gpu, oracle):
    g = golden("quant")
    for n in list(g["ns"]) + ["zero", "ties"]:
        q, s = gpu.qrow_i8(g[f"x{n}"])
        assert same_bits(q, g[f"q{n}"]) and s[0] == g[f"s{n}"], n
    rng = np.random.default_rng(2)
    for n in (5, 64, 1024, 3840, 15360, 16384):
        x = (rng.standard_normal((7, n)) * rng.choice([1e-4, 1, 300], (7, 1))).astype(np.float32)
        q, s = gpu.qrow_i8(x)
        qo, so = oracle.qrows_i8(x)
        assert same_bits(q, qo) and same_bits(s, so), n


def test_quant_g32_bit_exact(gpu, oracle):
    g = golden("quant")
    xq, xs, xsum = gpu.quant_g32(g["g32_x"])
    assert same_bits(xq, g["g32_q"]) and same_bits(xs, g["g32_s"]) and same_bits(xsum, g["g32_sum"])
    x = np.random.default_rng(3).standard_normal((33, 2048)).astype(np.float32)
    a, b = gpu.quant_g32(x), oracle.quant_g32(x)
    assert all(same_bits(u, v) for u, v in zip(a, b))


def test_weight_quantizers_bit_exact(gpu, oracle):
    for tag in "abc":
        g = golden("matmul_" + tag)
        q, s = gpu.quantize_rows(g["Wf"])
        assert same_bits(q, g["q8"]) and same_bits(s, g["s8"])
        q4, s16 = gpu.pack_q4r4(g["Wf"])
        assert same_bits(q4, g["q4"]) and same_bits(s16, g["s16"])
    rng = np.random.default_rng(4)
    W = (rng.standard_normal((203, 3072)) * 0.02).astype(np.float32)
    W[5, 64:96] = 0; W[7, 0:32] = np.abs(W[7, 0:32]); W[9, 32:64] = -np.abs(W[9, 32:64])
    a, b = gpu.pack_q4r4(W), oracle.pack_q4r4(W)
    assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])
    a, b = gpu.quantize_rows(W), oracle.quantize_rows(W)
    assert same_bits(a[0], b[0]) and same_bits(a[1], b[1])


def test_router_bit_exact_on_identical_probabilities(gpu, oracle):
    """tests/moe_tests.c:15-39: top-K over identical f32 inputs is bit-identical."""
    g = golden("router")
    for tag in "abcd":
        K = int(g[f"K_{tag}"])
        idx, w = gpu.moe_topk(g[f"p_{tag}"], K, 0)
        assert same_bits(idx, g[f"idx0_{tag}"]) and same_bits(w, g[f"w0_{tag}"])
        idx, w = gpu.moe_topk(g[f"p_{tag}"], K, 1)
        io, wo = oracle.moe_topk(g[f"p_{tag}"], K, 1)
        assert same_bits(idx, io) and same_bits(w, wo)
    rng = np.random.default_rng(5)
    for _ in range(50):
        E = int(rng.integers(2, 600)); K = int(rng.integers(1, min(E, 64) + 1))
        p = rng.random((3, E)).astype(np.float32); p[1, : E // 2] = p[1, 0]     # ties
        idx, w = gpu.moe_topk(p, K, 0)
        io, wo = oracle.moe_topk(p, K, 0)
        assert same_bits(idx, io) and same_bits(w, wo), (E, K)


def test_route_topk_indices_match_cpu(gpu, oracle):
    """softmax + top-K from logits: indices must equal the CPU's on every row;
    probabilities agree to one ulp (exp is correctly rounded here, libm's is not)."""
    g = golden("router")
    for tag in "abcd":
        K = int(g[f"K_{tag}"])
        idx, w, probs = gpu.route_topk(g[f"lg_{tag}"], K, want_probs=True)
        assert same_bits(idx, g[f"idx_{tag}"]), tag
        np.testing.assert_allclose(probs, g[f"p_{tag}"], rtol=3e-7, atol=0)
        np.testing.assert_allclose(w, g[f"w_{tag}"], rtol=1e-6, atol=0)
    rng = np.random.default_rng(6)
    for sd in (0.05, 1.0):
        lg = (rng.standard_normal((20000, 128)) * sd).astype(np.float32)
        idx, _ = gpu.route_topk(lg, 8)
        io, _, _ = oracle.route_topk(lg, 8)
        assert np.array_equal(idx, io), f"{(idx != io).any(axis=1).sum()} rows differ at sd={sd}"


@pytest.mark.parametrize("fmt", ["q8_0", "q4r4"])
@pytest.mark.parametrize("S", [1, 3])
def test_head_argmax(gpu, oracle, fmt, S):
    """lm_head + greedy pick in one call equals the reference's mat_apply followed by moty_argmax_v
    (nn/head.c:134-135, nn/sample.c:9-13): same ids, same logits; ties resolve to the first index."""
    rng = np.random.default_rng(S + len(fmt))
    V, D = 50304, 1024
    x = rng.standard_normal((S, D)).astype(np.float32)
    if fmt == "q8_0":
        Wq = rng.integers(-127, 128, (V, D), dtype=np.int8); sc = rng.uniform(0.001, 0.02, V).astype(np.float32)
        Wq[4000] = Wq[77]; sc[4000] = sc[77]            # two identical rows: equal logits
        W = gpu.Mat.i8(Wq, sc); lo = oracle.matmul_q_s(x, Wq, sc)
    else:
        Wf = (rng.standard_normal((V, D)) * 0.02).astype(np.float32)
        q4, s16 = oracle.pack_q4r4(Wf)
        W = gpu.Mat.q4r4(q4, s16, V, D); lo = oracle.matmul_q4r4_s(x, q4, s16, V)
    ids, lg = gpu.head_argmax(W, x, want_logits=True)
    assert same_bits(lg, lo)
    assert [int(i) for i in ids] == [oracle.argmax(lo[s]) for s in range(S)]
    assert np.array_equal(gpu.head_argmax(W, x), ids)


def test_argmax(gpu, oracle):
    g = golden("router")
    assert gpu.argmax(g["argmax_v"]) == int(g["argmax_i"])
    rng = np.random.default_rng(7)
    for n in (1, 2, 255, 50304, 151936, 262144):
        v = rng.standard_normal(n).astype(np.float32)
        if n > 10:
            v[n // 3] = v[n // 2] = v.max() + 1
        assert gpu.argmax(v) == oracle.argmax(v), n
