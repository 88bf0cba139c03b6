"""GPU parity of the tensor-core Q8_0 GEMM (S >= 16) through the C ABI: int32
accumulators and f32 outputs bit-exact against the oracle, plus size-independent
properties at the sweep's full sizes."""
import numpy as np
import pytest

from conftest import same_bits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("O,I", [(128, 128), (256, 1024), (1000, 1024), (130, 3072), (515, 3840), (64, 15360), (300, 144), (77, 2064), (9600, 256)])
@pytest.mark.parametrize("S", [16, 17, 32, 48, 64, 100, 128, 200, 256, 300, 512])
def test_q8_gemm_vs_oracle(gpu, oracle, O, I, S):
    rng = np.random.default_rng(O + 31 * I + S)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y, acc = gpu.mat_apply(gpu.Mat.i8(Wq, sc), x, want_acc=True)
    yo, acco = oracle.matmul_q_s(x, Wq, sc, want_acc=True)
    assert np.array_equal(acc, acco), f"{(acc != acco).sum()} accumulators differ"
    assert same_bits(y, yo)


def test_q8_gemm_extreme_values(gpu, oracle):
    """|acc| at its maximum: all weights -128, all activations saturating to -127."""
    O, I, S = 128, 16384, 16
    Wq = np.full((O, I), -128, np.int8); sc = np.ones(O, np.float32)
    x = np.full((S, I), -3.0, np.float32)
    y, acc = gpu.mat_apply(gpu.Mat.i8(Wq, sc), x, want_acc=True)
    assert (acc == 128 * 127 * I).all()


def test_batch_equals_rows_at_full_size(gpu):
    """Size-independent property at the sweep's largest shape: an S=512 batch through
    the tensor cores equals, bit for bit, the same rows through the decode GEMV
    (tests/qwen_tests.c:82-109 states the invariance for S=4)."""
    rng = np.random.default_rng(0)
    O, I, S = 151936, 1024, 512
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((S, I)).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc)
    yb = gpu.mat_apply(W, x)
    for s in (0, 1, 255, 511):
        assert same_bits(gpu.mat_apply(W, x[s:s + 1])[0], yb[s])
    # linearity of the integer part: doubling an activation row keeps its codes (the scale doubles)
    y2 = gpu.mat_apply(W, 2 * x[:16])
    assert same_bits(y2, 2 * yb[:16])


@pytest.mark.parametrize("O,I,S", [(19000, 2048, 300), (19100, 384, 300)])
def test_q8_gemm_256_row_tiles_vs_oracle(gpu, oracle, O, I, S):
    """Shapes with enough 256 x 256 tiles to take the two-accumulator variant, ragged in O and S."""
    rng = np.random.default_rng(O + I + S)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((S, I)).astype(np.float32)
    y, acc = gpu.mat_apply(gpu.Mat.i8(Wq, sc), x, want_acc=True)
    yo, acco = oracle.matmul_q_s(x, Wq, sc, want_acc=True)
    assert np.array_equal(acc, acco), f"{(acc != acco).sum()} accumulators differ"
    assert same_bits(y, yo)
