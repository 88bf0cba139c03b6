"""GPU: the sharded paths against the unsharded ones, one process per GPU over NCCL.
Runs with as many ranks as there are GPUs (up to 2 here); with a single GPU the
exchange still runs, to itself."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import moty_b200 as mb
        from moty_b200.parallel import ExpertParallelMoe, RowShardedMat
        if world > 1:
            mb.init([(rank + 1) % world])                    # another GPU first: entries without a handle must
        mb.init([rank])                                      # follow their pointers, not "the first device"
        dev = torch.device("cuda", rank)
        rng = np.random.default_rng(7)                       # same data on every rank

        # ---- row shards + all-gather: bit-identical to the whole matrix ----
        for (O, I, S) in ((1000, 1024, 1), (1000, 1024, 5), (3072, 1024, 32)):
            Wq = rng.integers(-127, 128, (O, I), dtype=np.int8); sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
            x = rng.standard_normal((S, I)).astype(np.float32)
            whole = mb.mat_apply(mb.Mat.i8(Wq, sc, device=rank), x)
            sh = RowShardedMat(mb.WF_I8, Wq, sc, O, I, device=rank)
            y = sh.apply(torch.from_numpy(x).to(dev))
            torch.cuda.synchronize()
            assert y.cpu().numpy().tobytes() == whole.tobytes(), f"row shards differ at {O}x{I} S={S}"
            if S == 1:                                       # the decode form: slice written in place, one all-gather
                for _ in range(2):
                    y1 = sh.decode(torch.from_numpy(x).to(dev))
                    torch.cuda.synchronize()
                    assert y1[:, :O].cpu().numpy().tobytes() == whole.tobytes(), "row-shard decode differs"

        # ---- expert parallel: tokens sharded, experts sharded, result bit-identical ----
        E, K, I, D, S_total = 8, 2, 64, 128, 13          # (with 2 ranks: 4 experts each)
        g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
        d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
        gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
        ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
        x_all = rng.standard_normal((S_total, D)).astype(np.float32)
        lg_all = (rng.standard_normal((S_total, E)) * 0.7).astype(np.float32)
        ref = mb.Moe(E, K, I, D, device=rank)
        ep = ExpertParallelMoe(E, K, I, D, device=rank)
        for e in range(E):
            ref.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
            ep.upload_expert(e, g[e], gs[e], u[e], us[e], d[e], ds[e])
        cut = S_total // world + (1 if world > 1 else 0)
        mine = slice(0, cut) if rank == 0 else slice(cut, S_total)
        for order, whole in ((1, ref.batch(x_all, lg_all)), (0, ref.olmoe(x_all, lg_all, 1))):
            out = ep.forward(torch.from_numpy(x_all[mine]).to(dev), torch.from_numpy(lg_all[mine]).to(dev), order=order)
            torch.cuda.synchronize()
            assert out.cpu().numpy().tobytes() == whole[mine].tobytes(), f"expert-parallel result differs (order {order})"
        # ---- the routes without a host-side plan ----
        # decode: the same token on every rank, one all-reduce of the [K][D] row table -> the one-GPU bits
        for t in range(3):
            x1, l1 = x_all[t:t + 1], lg_all[t:t + 1]
            out = ep.decode(torch.from_numpy(x1).to(dev), torch.from_numpy(l1).to(dev))
            torch.cuda.synchronize()
            assert out.cpu().numpy().tobytes() == ref.d1(x1, l1).tobytes(), "expert-parallel decode differs"
        # the same decode with the exchange over peer memory (the library's own kernels, no collective): several steps in
        # a row, the tables alternate, the step counter moves on every rank alike
        for t in range(5):
            x1, l1 = x_all[t:t + 1], lg_all[t:t + 1]
            out = ep.decode_peer(torch.from_numpy(x1).to(dev), torch.from_numpy(l1).to(dev))
            torch.cuda.synchronize()
            assert mb.lib().moty_cuda_kernel_status(rank, None) == 0, mb.lib().moty_cuda_last_error()
            assert out.cpu().numpy().tobytes() == ref.d1(x1, l1).tobytes(), f"peer-memory expert-parallel decode differs at step {t}"
        # prefill: all-gather + partial sums + reduce-scatter (sum over ranks in the collective's order: 1e-5)
        s_each = 6
        xs, ls = x_all[:world * s_each], lg_all[:world * s_each]
        whole = ref.batch(xs, ls)
        mine2 = slice(rank * s_each, (rank + 1) * s_each)
        out = ep.forward_gathered(torch.from_numpy(xs[mine2]).to(dev), torch.from_numpy(ls[mine2]).to(dev), order=1)
        torch.cuda.synchronize()
        assert np.abs(out.cpu().numpy() - whole[mine2]).max() <= 1e-5 * np.abs(whole).max()

        # ---- Q4R4 experts, decode route ----
        E4, K4, I4, D4 = 16, 4, 96, 128
        mk = lambda n: (rng.integers(0, 256, n * 64, dtype=np.uint8), rng.uniform(0.001, 0.01, n * 4).astype(np.float16).view(np.uint16))
        ng, nd = (I4 // 4) * (D4 // 32), (D4 // 4) * (I4 // 32)
        ref4 = mb.Moe(E4, K4, I4, D4, efmt=mb.WF_Q4R4, device=rank)
        ep4 = ExpertParallelMoe(E4, K4, I4, D4, efmt=mb.WF_Q4R4, device=rank)
        for e in range(E4):
            (g4, gs4), (u4, us4), (d4, ds4) = mk(ng), mk(ng), mk(nd)
            ref4.upload_expert(e, g4, gs4, u4, us4, d4, ds4); ep4.upload_expert(e, g4, gs4, u4, us4, d4, ds4)
        for t in range(3):
            x1 = rng.standard_normal((1, D4)).astype(np.float32); l1 = (rng.standard_normal((1, E4)) * 0.7).astype(np.float32)
            out = ep4.decode(torch.from_numpy(x1).to(dev), torch.from_numpy(l1).to(dev))
            torch.cuda.synchronize()
            assert out.cpu().numpy().tobytes() == ref4.d1(x1, l1).tobytes(), "expert-parallel Q4R4 decode differs"
            out = ep4.decode_peer(torch.from_numpy(x1).to(dev), torch.from_numpy(l1).to(dev))
            torch.cuda.synchronize()
            assert out.cpu().numpy().tobytes() == ref4.d1(x1, l1).tobytes(), "peer-memory Q4R4 decode differs"
    finally:
        dist.destroy_process_group()


def test_sharded_paths_match_unsharded():
    import torch
    import torch.multiprocessing as mp
    world = min(2, torch.cuda.device_count())
    assert world >= 1
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
