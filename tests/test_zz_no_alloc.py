"""GPU: the allocation-free Q8_0 entry against the ordinary one, through the C ABI.

The entry serves hosts that cannot let a library allocate device memory while
they run (they own the whole memory budget, or cannot stall on cudaMalloc), so
its scratch is a fixed array inside the library.  This file is named to be
collected last: if it fails, every other test has already run.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_pair(gpu, torch, O, I, S, seed):
    rng = np.random.default_rng(seed)
    Wq = rng.integers(-127, 128, (O, I), dtype=np.int8)
    sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
    x = rng.standard_normal((S, I)).astype(np.float32)
    dev = torch.device("cuda", 0)
    # the caller's own device buffers (allocated by the caller, here through torch)
    q_d = torch.from_numpy(Wq).to(dev); s_d = torch.from_numpy(sc).to(dev); x_d = torch.from_numpy(x).to(dev)
    y_new = torch.full((S, O), float("nan"), device=dev)
    y_old = torch.full((S, O), float("nan"), device=dev)
    torch.cuda.synchronize()
    gpu.q8_apply_noalloc(y_new.data_ptr(), x_d.data_ptr(), q_d.data_ptr(), s_d.data_ptr(), S, I, O, 0, 0)
    W = gpu.Mat.i8(Wq, sc)
    gpu.mat_apply_dev(W, y_old.data_ptr(), x_d.data_ptr(), S, 0)
    torch.cuda.synchronize()
    gpu.sync(0)
    a, b = y_new.cpu().numpy(), y_old.cpu().numpy()
    assert not np.isnan(a).any()
    assert a.tobytes() == b.tobytes(), f"no-alloc entry differs from mat_apply_dev at O={O} I={I} S={S}"


def test_noalloc_matches_existing_entry_twice_in_a_row(gpu):
    import torch
    # two calls in a row with different shapes: the second must not see stale scratch of the first
    _run_pair(gpu, torch, 3072, 1024, 8, seed=1)
    _run_pair(gpu, torch, 515, 3840, 3, seed=2)
    _run_pair(gpu, torch, 64, 16384, 1, seed=3)


def test_noalloc_rejects_sizes_beyond_its_scratch(gpu):
    import torch
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    for (S, I) in ((9, 1024), (0, 1024), (1, 16400), (1, 100), (1, 32768)):
        with pytest.raises(gpu.MotyCudaError, match="q8_apply_noalloc"):
            gpu.q8_apply_noalloc(p, p, p, p, S, I, 4, 0, 0)
    # a weight pointer off the 16-byte grid (a sliced tensor) is refused on the host, before any launch: the product
    # kernel reads weights with 128-bit loads.  Likewise f32 pointers off the 4-byte grid.
    with pytest.raises(gpu.MotyCudaError, match="16-byte aligned"):
        gpu.q8_apply_noalloc(p, p, p + 1, p, 1, 16, 1, 0, 0)
    with pytest.raises(gpu.MotyCudaError, match="4-byte aligned"):
        gpu.q8_apply_noalloc(p + 2, p, p, p, 1, 16, 1, 0, 0)
    torch.cuda.synchronize()                              # nothing was launched, the context is intact
    assert float(t.sum()) == 0.0
