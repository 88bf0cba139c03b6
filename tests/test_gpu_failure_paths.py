"""GPU: the give-up path of the bounded waits, the status entry for device-resident callers, the scratch freeze and
the device-restoring entries.  No test here faults, traps or hangs a GPU: the expiry tests run the production wait
functions on something nobody completes with a limit of a few thousand polls (selftest.cu); each finishes in
milliseconds and leaves the context usable."""
import time

import numpy as np
import pytest

from conftest import same_bits

pytestmark = pytest.mark.gpu


def _small_moe(gpu, rng):
    E, K, I, D = 16, 4, 96, 160
    m = gpu.Moe(E, K, I, D)
    for e in range(E):
        m.upload_expert(e, rng.integers(-127, 128, (I, D), dtype=np.int8), rng.uniform(0.001, 0.02, I).astype(np.float32),
                        rng.integers(-127, 128, (I, D), dtype=np.int8), rng.uniform(0.001, 0.02, I).astype(np.float32),
                        rng.integers(-127, 128, (D, I), dtype=np.int8), rng.uniform(0.001, 0.02, D).astype(np.float32))
    return m, rng.standard_normal((1, D)).astype(np.float32), (rng.standard_normal((1, E)) * 0.5).astype(np.float32)


@pytest.mark.parametrize("which,what", [(0, "tensor-core GEMM"), (1, "grid barrier"), (2, "bulk-copy")])
def test_an_expired_wait_is_reported_once_and_the_next_call_works(gpu, which, what):
    L = gpu.lib()
    rng = np.random.default_rng(which)
    m, x, lg = _small_moe(gpu, rng)
    before = m.d1(x, lg)                                          # the one-launch decode kernel (uses the grid barrier)
    Wq = rng.integers(-127, 128, (300, 256), dtype=np.int8); sc = rng.uniform(0.001, 0.02, 300).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc); xb = rng.standard_normal((32, 256)).astype(np.float32)
    yb = gpu.mat_apply(W, xb)                                     # the tensor-core GEMM
    assert L.moty_cuda_kernel_status(0, None) == 0
    t0 = time.perf_counter()
    assert L.moty_cuda_selftest_expire_wait(0, which, None) == 0  # enqueued; the kernel gives up by itself
    rc = L.moty_cuda_kernel_status(0, None)
    dt = time.perf_counter() - t0
    assert rc == -6 and what in L.moty_cuda_last_error().decode(), L.moty_cuda_last_error().decode()   # MOTY_CUDA_EKERNEL
    assert dt < 1.0, f"the give-up path took {dt:.3f} s"
    assert L.moty_cuda_kernel_status(0, None) == 0                # reported once, then clear
    # the next ordinary calls succeed with the same bits: error words cleared, barrier counters back at zero
    assert same_bits(m.d1(x, lg), before)
    assert same_bits(gpu.mat_apply(W, xb), yb)
    assert L.moty_cuda_kernel_status(0, None) == 0


def test_host_pointer_entry_reports_an_expired_wait_itself(gpu):
    """moty_cuda_moe_d1 (host pointers) reads the error word after its own launch: an expiry left by an earlier kernel on
    the stream surfaces as MOTY_CUDA_EKERNEL from that call, and the call after it is clean."""
    L = gpu.lib()
    m, x, lg = _small_moe(gpu, np.random.default_rng(9))
    want = m.d1(x, lg)
    assert L.moty_cuda_selftest_expire_wait(0, 1, None) == 0
    with pytest.raises(gpu.MotyCudaError, match="grid barrier"):
        m.d1(x, lg)
    assert same_bits(m.d1(x, lg), want)


def test_scratch_freeze_refuses_to_move_buffers(gpu):
    L = gpu.lib()
    rng = np.random.default_rng(3)
    Wq = rng.integers(-127, 128, (256, 512), dtype=np.int8); sc = rng.uniform(0.001, 0.02, 256).astype(np.float32)
    W = gpu.Mat.i8(Wq, sc)
    small = rng.standard_normal((4, 512)).astype(np.float32)
    y = gpu.mat_apply(W, small)
    assert L.moty_cuda_scratch_freeze(0, 1) == 0
    try:
        assert same_bits(gpu.mat_apply(W, small), y)              # fits what is reserved
        with pytest.raises(gpu.MotyCudaError, match="frozen"):    # a batch far beyond anything run in this process
            gpu.mat_apply(W, rng.standard_normal((60000, 512)).astype(np.float32))
    finally:
        assert L.moty_cuda_scratch_freeze(0, 0) == 0
    assert gpu.mat_apply(W, rng.standard_normal((600, 512)).astype(np.float32)).shape == (600, 256)


def test_entries_leave_the_callers_device_current(gpu):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("one GPU: nothing to restore")
    gpu.init([0, 1])
    rng = np.random.default_rng(4)
    Wq = rng.integers(-127, 128, (64, 128), dtype=np.int8); sc = rng.uniform(0.001, 0.02, 64).astype(np.float32)
    W1 = gpu.Mat.i8(Wq, sc, device=1)
    torch.cuda.set_device(0)
    gpu.mat_apply(W1, rng.standard_normal((2, 128)).astype(np.float32))
    assert torch.cuda.current_device() == 0
    from ctypes import c_int, byref
    cur = c_int(-1)
    import ctypes
    rt = ctypes.CDLL("libcudart.so.12")
    assert rt.cudaGetDevice(byref(cur)) == 0 and cur.value == 0


def test_device_position_out_of_range_is_clamped_and_reported(gpu):
    """A replayed decode step whose device counter ran past the documented maximum must not store past the KV cache:
    the kernels clamp the position and set an error word that moty_cuda_kernel_status reports."""
    import torch
    L = gpu.lib()
    H, KV, hd, max_t = 4, 2, 64, 16
    a = gpu.Attn(H, KV, hd, max_t)
    f = lambda *sh: torch.randn(sh, device="cuda")
    q, k, v, ctx = f(1, H * hd), f(1, KV * hd), f(1, KV * hd), f(1, H * hd)
    guard = torch.zeros(4096, device="cuda")                     # memory allocated after the cache: stays untouched
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    sh = gpu.stream_handle(torch.cuda.current_stream())
    a.core_posdev(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, pos.data_ptr(), max_t - 1, stream=sh)
    torch.cuda.synchronize()
    assert L.moty_cuda_kernel_status(0, None) == 0
    pos.fill_(10 ** 6)
    a.core_posdev(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, pos.data_ptr(), max_t - 1, stream=sh)
    torch.cuda.synchronize()
    assert L.moty_cuda_kernel_status(0, None) == -6 and "position" in L.moty_cuda_last_error().decode()
    assert float(guard.abs().sum()) == 0.0 and torch.isfinite(ctx).all()
    a.close()
