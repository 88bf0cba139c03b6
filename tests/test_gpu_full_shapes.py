"""GPU parity at the op sweep's own sizes: all six matrices (out x in) of the Q8_0 / grouped-int4 sweep at 1, 16 and
512 activation rows, compared with the oracle through the C ABI.

The whole product runs on the GPU at full size; the oracle checks every output row where that takes
seconds, and a spread sample of weight rows (whole 4-row blocks for Q4R4) where it would take minutes.
An output row depends on its own weight row only, so a sampled row is checked exactly as in a full
comparison -- bit for bit, int32 accumulators included."""
import numpy as np
import pytest

from conftest import same_bits

pytestmark = pytest.mark.gpu

SHAPES = [(1024, 1024), (3072, 1024), (1024, 3072), (151936, 1024), (15360, 3840), (3840, 15360)]
ROWS = (1, 16, 512)


def _row_sample(O, budget, rng, block=1):
    """All rows when O <= budget, else first and last blocks plus a random spread, as sorted row indices."""
    nb = (O + block - 1) // block
    if nb * block <= budget:
        return np.arange(O)
    pick = set(range(4)) | set(range(nb - 4, nb)) | set(int(b) for b in rng.choice(nb, budget // block - 8, replace=False))
    rows = np.concatenate([np.arange(b * block, min((b + 1) * block, O)) for b in sorted(pick)])
    return rows


@pytest.mark.parametrize("O,I", SHAPES)
def test_q8_full_shape(gpu, oracle, O, I):
    rng = np.random.default_rng(0)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8)
    sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc)
    for S in ROWS:
        x = rng.standard_normal((S, I)).astype(np.float32)
        y, acc = gpu.mat_apply(W, x, want_acc=True)
        rows = _row_sample(O, 4096 if S == 512 else 1 << 30, rng)
        yo, acco = oracle.matmul_q_s(x, np.ascontiguousarray(Wq[rows]), sc[rows], want_acc=True)
        assert np.array_equal(acc[:, rows], acco), (O, I, S)
        assert same_bits(np.ascontiguousarray(y[:, rows]), yo), (O, I, S)
        assert same_bits(gpu.mat_apply(W, x), y)            # the entry without accumulators takes the same path


@pytest.mark.parametrize("O,I", SHAPES)
def test_q4r4_full_shape(gpu, oracle, O, I):
    rng = np.random.default_rng(0)
    nb, ng = O // 4, I // 32
    # random nibble codes and f16 scales in the range the packer produces for N(0, 0.02) weights: packing 156 M weights
    # on the CPU takes minutes, and the product does not care where the codes came from
    q4 = rng.integers(0, 256, (nb, ng * 64), dtype=np.uint8)
    s16 = rng.uniform(0.002, 0.012, (nb, ng * 4)).astype(np.float16).view(np.uint16)
    W = gpu.Mat.q4r4(q4.reshape(-1), s16.reshape(-1), O, I)
    for S in ROWS:
        x = rng.standard_normal((S, I)).astype(np.float32)
        y = gpu.mat_apply(W, x)
        budget = {1: 1 << 30, 16: 16384, 512: 512}[S] if O * I > (1 << 24) else 1 << 30
        rows = _row_sample(O, budget, rng, block=4)
        blocks = rows[::4] // 4
        yo = oracle.matmul_q4r4_s(x, np.ascontiguousarray(q4[blocks]).reshape(-1), np.ascontiguousarray(s16[blocks]).reshape(-1), len(rows))
        got = np.ascontiguousarray(y[:, rows])
        if S <= 4:
            assert same_bits(got, yo), (O, I, S, float(np.abs(got - yo).max()))
        else:
            assert same_bits(got, yo) or np.abs(got - yo).max() <= 1e-5 * np.abs(yo).max(), (O, I, S, float(np.abs(got - yo).max()))
