"""GPU parity of mat_apply (Q8_0, Q4R4, per-row int4) through the C ABI."""
import numpy as np
import pytest

from conftest import golden, same_bits

pytestmark = pytest.mark.gpu

S_ALL = (1, 2, 3, 4, 5, 7, 16, 37)


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_q8_golden_bit_exact(gpu, oracle, tag):
    g = golden("matmul_" + tag)
    W = gpu.Mat.i8(g["W8"], g["sc"])
    for S in S_ALL:
        y, acc = gpu.mat_apply(W, g[f"x{S}"], want_acc=True)
        _, acc_o = oracle.matmul_q_s(g[f"x{S}"], g["W8"], g["sc"], want_acc=True)
        assert np.array_equal(acc, acc_o), f"int32 accumulators differ at S={S}"
        assert same_bits(y, g[f"y8_{S}"]), f"f32 outputs differ at S={S}"
        assert same_bits(gpu.mat_apply(W, g[f"x{S}"]), g[f"y8_{S}"])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_q4r4_golden_bit_exact(gpu, tag):
    g = golden("matmul_" + tag)
    O, I = int(g["O"]), int(g["I"])
    W = gpu.Mat.q4r4(g["q4"], g["s16"], O, I)
    for S in S_ALL:
        y = gpu.mat_apply(W, g[f"x{S}"])
        assert same_bits(y, g[f"y4_{S}"]), f"S={S}: max diff {np.abs(y - g[f'y4_{S}']).max()}"


@pytest.mark.parametrize("O,I", [(1024, 1024), (3072, 1024), (1024, 3072), (515, 3840), (260, 15360), (77, 16384), (9, 16), (5, 100)])
@pytest.mark.parametrize("S", [1, 2, 4, 8, 16, 33])
def test_q8_vs_oracle(gpu, oracle, O, I, S):
    """Config-2 recipe: int8 U[-127,127], scales U(0.001,0.02), x ~ N(0,1)."""
    rng = np.random.default_rng(O * 7 + I + S)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((S, I)).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc)
    y, acc = gpu.mat_apply(W, x, want_acc=True)
    yo, acco = oracle.matmul_q_s(x, Wq, sc, want_acc=True)
    assert np.array_equal(acc, acco)
    assert same_bits(y, yo)


@pytest.mark.parametrize("O,I,S", [(1024, 3072, 16), (515, 3840, 9), (2000, 4096, 12), (5121, 6912, 12), (3000, 2176, 16)])
def test_q8_small_batch_split_k(gpu, oracle, O, I, S):
    """9..16 rows against matrices with few 128-row tiles: the MMA kernel splits K over several CTAs whose int32
    partials meet in a scratch table that has to be zero again afterwards -- so every case runs twice, the second
    time on other activations.  Row counts off the tile size, a row length that is not a multiple of the 128-byte stage."""
    rng = np.random.default_rng(O + I * 3 + S)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc)
    for _ in range(2):
        x = rng.standard_normal((S, I)).astype(np.float32)
        y, acc = gpu.mat_apply(W, x, want_acc=True)
        yo, acco = oracle.matmul_q_s(x, Wq, sc, want_acc=True)
        assert np.array_equal(acc, acco)
        assert same_bits(y, yo)


@pytest.mark.parametrize("O,I", [(1024, 1024), (3072, 1024), (1022, 3072), (515, 3840), (258, 15360), (768, 2048), (4, 32), (7, 64)])
@pytest.mark.parametrize("S", [1, 2, 3, 4, 7, 12, 37])
def test_q4r4_vs_oracle(gpu, oracle, O, I, S):
    rng = np.random.default_rng(O * 3 + I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, s16 = oracle.pack_q4r4(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    W = gpu.Mat.q4r4(q4, s16, O, I)
    y = gpu.mat_apply(W, x)
    yo = oracle.matmul_q4r4_s(x, q4, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I,S", [(4096, 256, 320), (4096, 352, 157), (4100, 96, 163), (2052, 3840, 33), (4096, 64, 321)])
def test_q4r4_batches_vs_oracle(gpu, oracle, O, I, S):
    """Batches large enough for the 16- and 32-token CTA tiles of the MMA kernel, ragged in every
    dimension: rows not a multiple of 128, tokens not a multiple of 8 (mixed 4-token / single-token
    formulas in the last tile), group counts that are not a multiple of the 8-group stage."""
    rng = np.random.default_rng(O + I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, s16 = oracle.pack_q4r4(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.q4r4(q4, s16, O, I), x)
    yo = oracle.matmul_q4r4_s(x, q4, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I,S", [(4096, 256, 320), (4100, 352, 157), (2052, 3840, 37), (1024, 1024, 5), (515, 3840, 512)])
def test_q4r4_batch_relaxed(gpu, oracle, O, I, S):
    """moty_cuda_set_q4r4_batch_relaxed(1): the token-by-token formula (hw/hw_q4r4.h:58-59) for every token of a batch.
    Tokens that moty_matmul_q4r4_s sends through that formula -- the last S % 4 of the batch's final 32-token tile
    (nn/matmul.c:424-432) -- keep their bits; the others stay within 1e-5 of the row's magnitude.
    Q8R4 has one formula, so its relaxed result is bit for bit the exact one.  The switch is put back and the exact path
    checked again afterwards."""
    rng = np.random.default_rng(O + 7 * I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, s16 = oracle.pack_q4r4(Wf)
    q8, s16b = oracle.pack_q8r4(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    W4, W8 = gpu.Mat.q4r4(q4, s16, O, I), gpu.Mat.q8r4(q8, s16b, O, I)
    yo = oracle.matmul_q4r4_s(x, q4, s16, O)
    L = gpu.lib()
    prev = L.moty_cuda_set_q4r4_batch_relaxed(1)
    try:
        y = gpu.mat_apply(W4, x)
        y8 = gpu.mat_apply(W8, x)
    finally:
        assert L.moty_cuda_set_q4r4_batch_relaxed(prev) == 1
    assert prev == 0
    tile0 = (S - 1) // 32 * 32
    first_single = tile0 + (S - tile0) // 4 * 4                             # tokens from here on take the token-by-token kernel
    assert same_bits(y[first_single:], yo[first_single:])
    err = np.abs(y - yo).max(axis=1) / np.abs(yo).max(axis=1)
    assert err.max() <= 1e-5, err.max()
    assert first_single == 0 or err[:first_single].max() > 0, "the relaxed kernel did not run"
    assert same_bits(y8, oracle.matmul_q8r4_s(x, q8, s16b, O))
    assert same_bits(gpu.mat_apply(W4, x), yo)                              # the default again


@pytest.mark.parametrize("O,I", [(57000, 256), (56833, 512), (151936, 1024)])
def test_q4r4_decode_many_rows_vs_oracle(gpu, oracle, O, I):
    """Matrices with enough rows for the lane-per-row decode kernel (one activation row), a row
    count that is not a multiple of 32, and the vocabulary shape of the benchmark."""
    rng = np.random.default_rng(O + I)
    q4 = rng.integers(0, 256, (O + 3) // 4 * (I // 32) * 64, dtype=np.uint8)
    s16 = rng.uniform(0.001, 0.01, (O + 3) // 4 * (I // 32) * 4).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((1, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.q4r4(q4, s16, O, I), x)
    yo = oracle.matmul_q4r4_s(x, q4, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I", [(15360, 3840), (9601, 5504), (3838, 15360), (4001, 12800), (3199, 16384), (3200, 16352),
                                 (30001, 2048), (28417, 1920)])
def test_q4r4_decode_few_long_rows_vs_oracle(gpu, oracle, O, I):
    """One activation row against matrices with too few rows for the lane-per-row kernel.  The first six take the
    two-phase kernel (integer sums in parallel, then the chain from a table of factors): the FFN shapes of the
    benchmark, row counts that are not multiples of 4 or 32, group counts that are not multiples of the 32-group
    slab, the longest row allowed and an odd group count.  The last two have a middling row count and take the
    kernel fed by bulk copies."""
    rng = np.random.default_rng(O + I)
    q4 = rng.integers(0, 256, (O + 3) // 4 * (I // 32) * 64, dtype=np.uint8)
    s16 = rng.uniform(0.001, 0.01, (O + 3) // 4 * (I // 32) * 4).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((1, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.q4r4(q4, s16, O, I), x)
    yo = oracle.matmul_q4r4_s(x, q4, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I", [(1024, 1024), (1022, 3072), (515, 3840), (258, 15360), (4, 32), (7, 96), (4100, 352)])
@pytest.mark.parametrize("S", [1, 2, 4, 7, 12, 37, 163])
def test_q8r4_vs_oracle(gpu, oracle, O, I, S):
    """Q8R4 (the int8 sibling of Q4R4): every batch size through the MMA kernel, ragged rows, tokens and groups."""
    rng = np.random.default_rng(O * 5 + I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q8, s16 = oracle.pack_q8r4(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.q8r4(q8, s16, O, I), x)
    yo = oracle.matmul_q8r4_s(x, q8, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I", [(15360, 3840), (3838, 15360), (9601, 5504), (3200, 16352), (56833, 512)])
def test_q8r4_decode_large_vs_oracle(gpu, oracle, O, I):
    """One activation row against large Q8R4 matrices (the two-phase decode kernel): FFN shapes, row counts that are
    not multiples of 4 or 32, group counts that are not multiples of the 16-group slab, an odd group count, many
    short rows."""
    rng = np.random.default_rng(O * 3 + I)
    q8 = rng.integers(-127, 128, (O + 3) // 4 * (I // 32) * 128, dtype=np.int8)
    s16 = rng.uniform(0.001, 0.01, (O + 3) // 4 * (I // 32) * 4).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((1, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.q8r4(q8, s16, O, I), x)
    yo = oracle.matmul_q8r4_s(x, q8, s16, O)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


def test_q8r4_golden_and_extremes(gpu, oracle):
    g = golden("matmul_q8r4")
    for tag in ("a", "b"):
        O = int(g[f"O_{tag}"])
        for S in (1, 5, 37):
            assert same_bits(gpu.matmul_q8r4_s(g[f"x_{tag}_{S}"], g[f"q8_{tag}"], g[f"s16_{tag}"], O), g[f"y_{tag}_{S}"])
    O, I = 8, 16384                                           # extreme codes and activations, the longest row
    q8 = np.full(2 * (I // 32) * 128, -128, np.int8)
    s16 = np.full(2 * (I // 32) * 4, 0x3C00, np.uint16)      # scale 1.0
    x = np.full((2, I), 127.0, np.float32); x[1] = -127.0
    assert same_bits(gpu.mat_apply(gpu.Mat.q8r4(q8, s16, O, I), x), oracle.matmul_q8r4_s(x, q8, s16, O))


def test_q4r4_long_rows_and_int16_worst_case(gpu, oracle):
    """tests/q4r4_tests.c:88-172: extreme codes and activations, long rows."""
    O, I = 8, 16384
    q4 = np.full(2 * (I // 32) * 64, 0xFF, np.uint8)            # every code 15
    s16 = np.full(2 * (I // 32) * 4, 0x3C00, np.uint16)          # scale 1.0
    x = np.full((2, I), 127.0, np.float32); x[1] = -127.0
    W = gpu.Mat.q4r4(q4, s16, O, I)
    assert same_bits(gpu.mat_apply(W, x), oracle.matmul_q4r4_s(x, q4, s16, O))


def test_i4_rows(gpu, oracle):
    """Per-row int4 (WF_I4): held on the device as the int8 codes nibble - 8, so one row goes through the streaming
    GEMV, small batches through the mma.sync kernel and large ones through the tcgen05 GEMM -- all bit for bit
    moty_matmul_i4_s with IDOT4=1; odd row lengths, row shards, and the format the handle reports."""
    rng = np.random.default_rng(9)
    for (O, I, S) in ((64, 128, 1), (33, 101, 3), (1024, 1024, 1), (1024, 1024, 5), (1000, 4096, 12), (1024, 1024, 64),
                      (515, 3840, 512), (300, 15360, 9), (77, 16384, 2)):
        Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
        q4, sc = oracle.pack_int4(Wf)
        x = rng.standard_normal((S, I)).astype(np.float32)
        W = gpu.Mat.i4(q4, sc, O, I)
        assert same_bits(gpu.mat_apply(W, x), oracle.matmul_i4_idot_s(x, q4, sc, I)), (O, I, S)
    O, I = 1000, 1024
    q4 = rng.integers(0, 256, (O, I // 2), dtype=np.uint8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((3, I)).astype(np.float32)
    W = gpu.Mat.i4(q4, sc, O, I)
    whole = gpu.mat_apply(W, x)
    assert same_bits(whole, oracle.matmul_i4_idot_s(x, q4, sc, I))
    parts = [gpu.mat_apply(gpu.Mat.i4(q4, sc, O, I, rows=(a, b)), x) for a, b in ((0, 252), (252, 501), (501, 1000))]
    assert same_bits(np.concatenate(parts, axis=1), whole)
    import ctypes as C
    fmt = C.c_int(-1)
    assert gpu.lib().moty_cuda_mat_shape(W.h, C.byref(fmt), None, None, None) == 0 and fmt.value == gpu.WF_I4
    assert W.nbytes() == O * I + 4 * O


@pytest.mark.parametrize("O,I", [(1024, 1024), (3072, 1024), (1022, 3072), (515, 3840), (258, 15360), (77, 16384), (5, 32), (300, 96)])
@pytest.mark.parametrize("S", [1, 2, 3, 4, 7, 8, 19])
def test_i4g_vs_oracle(gpu, oracle, O, I, S):
    """WF_I4G (grouped int4, group 32, f32 group scales), integer path: ragged rows and token tiles, the longest row.
    Row lengths that are not a multiple of 64 take the f32 x int4 product, as in the reference (nn/matmul.c:172)."""
    rng = np.random.default_rng(O * 11 + I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, sc = oracle.pack_int4_grouped(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.i4g(q4, sc, O, I), x)
    if I % 64:
        yo = oracle.matmul_i4g_f32_s(x, q4, sc)
        assert np.abs(y - yo).max() <= 2e-6 * np.abs(yo).max()
        return
    yo = oracle.matmul_i4g_idot_s(x, q4, sc)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"


@pytest.mark.parametrize("O,I,S", [(4096, 256, 320), (4100, 320, 157), (2052, 3840, 33), (1000, 64, 9), (515, 192, 70), (130, 16384, 12),
                                   (3838, 15360, 19), (1024, 1024, 512)])
def test_i4g_batches_vs_oracle(gpu, oracle, O, I, S):
    """WF_I4G batches of nine rows and more (the tensor-core kernel, one integer MMA per group): ragged in every dimension
    -- rows not a multiple of 128, tokens not a multiple of 8, group counts below and not a multiple of the 8-group
    stage -- and codes at both extremes with saturating activations.  Bit-exact."""
    rng = np.random.default_rng(O + 3 * I + S)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, sc = oracle.pack_int4_grouped(Wf)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y = gpu.mat_apply(gpu.Mat.i4g(q4, sc, O, I), x)
    yo = oracle.matmul_i4g_idot_s(x, q4, sc)
    assert same_bits(y, yo), f"max diff {np.abs(y - yo).max()} of {np.abs(yo).max()}"
    if O <= 1100:
        for fill in (0x00, 0xFF):
            q4 = np.full((O, I // 2), fill, np.uint8); sc = rng.uniform(0.1, 0.5, (O, I // 32)).astype(np.float32)
            x = np.zeros((S, I), np.float32); x[0] = 1000.0; x[1, ::2] = -3.0; x[1, 1::2] = 3.0; x[3:] = rng.standard_normal((S - 3, I))
            assert same_bits(gpu.mat_apply(gpu.Mat.i4g(q4, sc, O, I), x), oracle.matmul_i4g_idot_s(x, q4, sc))


def test_i4g_golden_and_extremes(gpu, oracle):
    g = golden("matmul_i4g")
    for tag in ("a", "b"):
        q4, sc = g[f"q4_{tag}"], g[f"scale_{tag}"]
        O, I = q4.shape[0], q4.shape[1] * 2
        W = gpu.Mat.i4g(q4, sc, O, I)
        for S in (1, 2, 5, 9):
            assert same_bits(gpu.mat_apply(W, g[f"x_{tag}_{S}"]), g[f"y_{tag}_{S}"])
        assert same_bits(gpu.matmul_i4_grouped_s(g[f"x_{tag}_5"], q4, sc, O), g[f"y_{tag}_5"])
    # every code at an extreme, saturating activations, a zero row
    O, I = 64, 2048
    for fill in (0x00, 0xFF):
        q4 = np.full((O, I // 2), fill, np.uint8); sc = np.full((O, I // 32), 0.37, np.float32)
        x = np.zeros((3, I), np.float32); x[0] = 1000.0; x[1, ::2] = -3.0; x[1, 1::2] = 3.0
        assert same_bits(gpu.mat_apply(gpu.Mat.i4g(q4, sc, O, I), x), oracle.matmul_i4g_idot_s(x, q4, sc))


def test_host_weight_entries(gpu, oracle):
    g = golden("matmul_a")
    assert same_bits(gpu.matmul_q_s(g["x5"], g["W8"], g["sc"]), g["y8_5"])
    assert same_bits(gpu.matmul_q4r4_s(g["x5"], g["q4"], g["s16"], int(g["O"])), g["y4_5"])


def test_row_shards_concatenate_to_the_whole(gpu, oracle):
    """A matrix cut into row shards gives, concatenated, the unsharded result bit for bit."""
    rng = np.random.default_rng(10)
    O, I = 1000, 1024
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((3, I)).astype(np.float32)
    whole = gpu.mat_apply(gpu.Mat.i8(Wq, sc), x)
    parts = [gpu.mat_apply(gpu.Mat.i8(Wq, sc, rows=(a, b)), x) for a, b in ((0, 252), (252, 500), (500, 1000))]
    assert same_bits(np.concatenate(parts, axis=1), whole)
    Wf = (rng.standard_normal((O, I)) * 0.02).astype(np.float32)
    q4, s16 = oracle.pack_q4r4(Wf)
    whole = gpu.mat_apply(gpu.Mat.q4r4(q4, s16, O, I), x)
    parts = [gpu.mat_apply(gpu.Mat.q4r4(q4, s16, O, I, rows=(a, b)), x) for a, b in ((0, 252), (252, 500), (500, 1000))]
    assert same_bits(np.concatenate(parts, axis=1), whole)


def test_errors_are_loud(gpu):
    with pytest.raises(gpu.MotyCudaError):
        gpu.Mat.q4r4(np.zeros(64, np.uint8), np.zeros(4, np.uint16), 4, 40)          # I % 32 != 0
    W = gpu.Mat.i8(np.zeros((4, 32), np.int8), np.ones(4, np.float32))
    with pytest.raises(ValueError):
        gpu.mat_apply(W, np.zeros((1, 16), np.float32))
    with pytest.raises(gpu.MotyCudaError):
        gpu.Mat.i8(np.zeros((4, 32), np.int8), np.ones(4, np.float32), device=7)     # not initialised


def test_q8_multi_launch_equals_single_launches(gpu, oracle):
    """Several independent one-row products in one launch (moty_cuda_mat_apply_multi_dev): the bits of one
    mat_apply per matrix and of the oracle; rows shared between matrices (q, k, v of a layer); shapes from the sweep
    and ragged ones; twice in a row."""
    import torch
    rng = np.random.default_rng(5)
    shapes = [(1024, 1024), (3072, 1024), (1024, 3072), (515, 3840), (9, 16), (2048, 1024), (1, 4096), (259, 15360)]
    mats = [(rng.integers(-127, 128, s, dtype=np.int8), rng.uniform(0.001, 0.02, s[0]).astype(np.float32)) for s in shapes]
    W = [gpu.Mat.i8(q, sc) for q, sc in mats]
    sh = gpu.stream_handle(torch.cuda.current_stream())
    for trial in range(2):
        xs = [rng.standard_normal((1, s[1])).astype(np.float32) for s in shapes]
        xs[5] = xs[0]                                            # 2048x1024 shares the row of 1024x1024
        dx = [torch.from_numpy(x).cuda() for x in xs]
        dx[5] = dx[0]
        dy = [torch.full((1, s[0]), float("nan"), device="cuda") for s in shapes]
        gpu.mat_apply_multi_dev(W, [y.data_ptr() for y in dy], [x.data_ptr() for x in dx], sh)
        torch.cuda.synchronize()
        for (q, sc), w, x, y in zip(mats, W, xs, dy):
            got = y.cpu().numpy()
            assert same_bits(got, gpu.mat_apply(w, x)) and same_bits(got, oracle.matmul_q_s(x, q, sc))
    # rows longer than 4096 values are split in K: two such matrices in one launch (their cells sit side by side), twice
    shapes2 = [(300, 8192), (77, 4112), (64, 16384), (1000, 1024)]
    mats2 = [(rng.integers(-127, 128, s, dtype=np.int8), rng.uniform(0.001, 0.02, s[0]).astype(np.float32)) for s in shapes2]
    W2 = [gpu.Mat.i8(q, sc) for q, sc in mats2]
    for trial in range(2):
        xs = [rng.standard_normal((1, s[1])).astype(np.float32) for s in shapes2]
        dx = [torch.from_numpy(x).cuda() for x in xs]
        dy = [torch.full((1, s[0]), float("nan"), device="cuda") for s in shapes2]
        gpu.mat_apply_multi_dev(W2, [y.data_ptr() for y in dy], [x.data_ptr() for x in dx], sh)
        torch.cuda.synchronize()
        for (q, sc), w, x, y in zip(mats2, W2, xs, dy):
            got = y.cpu().numpy()
            assert same_bits(got, gpu.mat_apply(w, x)) and same_bits(got, oracle.matmul_q_s(x, q, sc))


def test_host_entry_with_pinned_buffers_equals_pageable(gpu, oracle):
    """moty_cuda_mat_apply with page-locked buffers at both ends moves x in and y out with kernels and waits on a flag
    word instead of synchronising the stream; with pageable buffers (or an odd alignment) it uses copy-engine transfers.
    Same bits either way, call after call, odd sizes included."""
    rng = np.random.default_rng(41)
    for (O, I, S) in ((1024, 1024, 1), (515, 3840, 1), (3, 16, 1), (4099, 1024, 3), (1000, 112, 8)):
        Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
        W = gpu.Mat.i8(Wq, sc)
        hx = gpu.pinned_empty((S, I), np.float32); hy = gpu.pinned_empty((S, O), np.float32)
        pad = gpu.pinned_empty((S * I + 1,), np.float32)                   # a pinned buffer 4 bytes off the 16-byte grid
        for rep in range(5):                                               # the third call on is a replayed graph of the call
            x = rng.standard_normal((S, I)).astype(np.float32)
            hx[...] = x; hy[...] = np.nan
            gpu.mat_apply(W, hx, hy)                                       # pinned -> kernels
            want = oracle.matmul_q_s(x, Wq, sc)
            assert hy.tobytes() == want.tobytes(), (O, I, S, rep)
            assert gpu.mat_apply(W, x).tobytes() == want.tobytes()         # pageable -> copies
            off = pad[1:].reshape(S, I); off[...] = x
            y2 = gpu.pinned_empty((S, O), np.float32)
            gpu.mat_apply(W, off, y2)                                      # misaligned pinned x -> copies
            assert y2.tobytes() == want.tobytes()
        # a matrix freed and another one created (possibly at the same address) must not meet a stale graph
        W.free()
        Wq2 = rng.integers(-127, 128, (O, I), dtype=np.int8); W2 = gpu.Mat.i8(Wq2, sc)
        for rep in range(3):
            gpu.mat_apply(W2, hx, hy)
            assert hy.tobytes() == oracle.matmul_q_s(np.asarray(hx), Wq2, sc).tobytes()


def test_i4g_float_path(gpu, oracle):
    """MOTY_WF_I4G through the reference's default product (f32 x int4, no activation quantizer) after
    moty_cuda_set_i4g_float_path(1): the reference's vectors and the oracle at 1e-6 of the output magnitude (a 32-term f32
    sum in another order); row lengths that are not a multiple of 64 take it under either setting, as in the reference;
    the default stays the bit-exact integer path."""
    g = golden("i4g_f32")
    L = gpu.lib()
    for t in "abc":
        x, q4, sc, want = g[f"x_{t}"], g[f"q4_{t}"], g[f"s_{t}"], g[f"y_{t}"]
        O, I = sc.shape[0], x.shape[1]
        W = gpu.Mat.i4g(q4, sc, O, I)
        prev = L.moty_cuda_set_i4g_float_path(1)
        y = gpu.mat_apply(W, x)
        L.moty_cuda_set_i4g_float_path(prev)
        assert np.abs(y - want).max() <= 1e-6 * np.abs(want).max(), t
        y0 = gpu.mat_apply(W, x)                                            # default setting
        if I % 64 == 0:
            assert y0.tobytes() == oracle.matmul_i4g_idot_s(x, q4, sc).tobytes()
        else:
            assert y0.tobytes() == y.tobytes()
    rng = np.random.default_rng(5)
    for (O, I, S) in ((1000, 4096, 1), (333, 2080, 9), (64, 16416, 2)):     # the last: longer than the integer path takes
        q4 = rng.integers(0, 256, (O, I // 2), dtype=np.uint8); sc = rng.uniform(0.001, 0.02, (O, I // 32)).astype(np.float32)
        x = rng.standard_normal((S, I)).astype(np.float32)
        W = gpu.Mat.i4g(q4, sc, O, I)
        prev = L.moty_cuda_set_i4g_float_path(1)
        y = gpu.mat_apply(W, x)
        L.moty_cuda_set_i4g_float_path(prev)
        want = oracle.matmul_i4g_f32_s(x, q4, sc)
        assert np.abs(y - want).max() <= 2e-6 * np.abs(want).max(), (O, I, S)
