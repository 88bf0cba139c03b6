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

        # ---- expert parallel: tokens sharded, experts sharded, result bit-identical ----
        E, K, I, D, S_total = 8, 2, 64, 128, 13
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
    finally:
        dist.destroy_process_group()


def test_sharded_paths_match_unsharded():
    import torch
    import torch.multiprocessing as mp
    world = min(2, torch.cuda.device_count())
    assert world >= 1
    mp.spawn(_worker, args=(world, _free_port()), nprocs=world, join=True)
