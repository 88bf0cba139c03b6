"""CPU, two gloo ranks: the host-side sharding logic (row ranges, the expert-parallel
dispatch plan, the two all-to-all exchanges and the un-permutation) with the CPU
oracle standing in for the three GPU compute steps."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def test_shard_rows():
    from moty_b200.parallel import shard_experts, shard_rows
    for O, world, align in ((1000, 3, 1), (1000, 8, 4), (151936, 8, 4), (7, 4, 4), (262144, 2, 1)):
        got = [shard_rows(O, world, r, align) for r in range(world)]
        covered = []
        for lo, hi, per in got:
            assert per % align == 0 and hi - lo <= per and (hi == lo or lo % align == 0)
            covered += list(range(lo, hi))
        assert covered == list(range(O))
    assert [shard_experts(64, 4, r) for r in range(4)] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        shard_experts(10, 4, 0)


def _make_layer(seed, E, K, I, D):
    rng = np.random.default_rng(seed)
    g = rng.integers(-127, 128, (E, I, D), dtype=np.int8); u = rng.integers(-127, 128, (E, I, D), dtype=np.int8)
    d = rng.integers(-127, 128, (E, D, I), dtype=np.int8)
    gs, us = (rng.uniform(0.001, 0.02, (E, I)).astype(np.float32) for _ in range(2))
    ds = rng.uniform(0.001, 0.02, (E, D)).astype(np.float32)
    return g, u, d, gs, us, ds


def _worker(rank, world, port, S_total, order):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moty_b200.parallel import ExpertParallelMoe
        from oracle import Experts, Oracle
        o = Oracle()
        E, K, I, D = 8, 2, 32, 64
        g, u, d, gs, us, ds = _make_layer(3, E, K, I, D)
        rng = np.random.default_rng(4)
        x_all = rng.standard_normal((S_total, D)).astype(np.float32)
        lg_all = (rng.standard_normal((S_total, E)) * 0.7).astype(np.float32)
        # ragged token shards: rank 0 gets one token more than an even split
        cut = S_total // world + 1
        mine = slice(0, cut) if rank == 0 else slice(cut, S_total)

        def route_fn(logits, K_, norm):
            idx, w, _ = o.route_topk(logits.numpy(), K_)
            return torch.from_numpy(idx), torch.from_numpy(w)

        lo, hi = rank * (E // world), (rank + 1) * (E // world)

        def expert_fn(rows, eids):
            out = np.zeros(rows.shape, np.float32)
            for i, e in enumerate(eids.tolist()):
                assert lo <= e < hi, "a row reached a rank that does not own its expert"
                xr = rows[i:i + 1].numpy()
                h = o.silu_mul(o.matmul_q_s(xr, g[e], gs[e]), o.matmul_q_s(xr, u[e], us[e]))
                out[i] = o.matmul_q_s(h, d[e], ds[e])[0]
            return torch.from_numpy(out)

        def combine_fn(h_sk, w, idx, order_):
            s, K_ = w.shape
            out = np.zeros((s, h_sk.shape[1]), np.float32)
            h = h_sk.numpy().reshape(s, K_, -1)
            for t in range(s):
                ks = list(range(K_))
                if order_ == 1:
                    ks.sort(key=lambda k: int(idx[t, k]))
                acc = np.zeros(h.shape[2], np.float64)
                for k in ks:                              # fused multiply-add per step, rounded to f32
                    acc = (np.float64(w[t, k].item()) * h[t, k].astype(np.float64) + acc).astype(np.float32).astype(np.float64)
                out[t] = acc.astype(np.float32)
            return torch.from_numpy(out)

        ep = ExpertParallelMoe(E, K, I, D, expert_fn=expert_fn, combine_fn=combine_fn, route_fn=route_fn)
        got = ep.forward(torch.from_numpy(x_all[mine]), torch.from_numpy(lg_all[mine]), order=order).numpy()
        ex = Experts(E, K, I, D, g, u, d, gs, us, ds)
        if order == 1:
            want = o.moe_batch(ex, x_all, lg_all)[0][mine]
        else:
            want = o.olmoe_moe(ex, x_all, lg_all, 1)[0][mine]
        np.testing.assert_allclose(got, want, rtol=2e-6, atol=1e-6 * np.abs(want).max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("order", [0, 1])
def test_expert_parallel_exchange_two_ranks(order):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 11, order), nprocs=2, join=True)


def _fixed_size_worker(rank, world, port):
    """The two routes without a host-side plan: replicated-token decode (all-reduce of the [K][D] row table, exact)
    and prefill by all-gather + reduce-scatter (f32 rounding)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moty_b200.parallel import ExpertParallelMoe
        from oracle import Experts, Oracle
        o = Oracle()
        E, K, I, D = 8, 3, 32, 64
        g, u, d, gs, us, ds = _make_layer(5, E, K, I, D)
        ex = Experts(E, K, I, D, g, u, d, gs, us, ds)
        lo, hi = rank * (E // world), (rank + 1) * (E // world)

        def expert_row(xr, e):
            h = o.silu_mul(o.matmul_q_s(xr, g[e], gs[e]), o.matmul_q_s(xr, u[e], us[e]))
            return o.matmul_q_s(h, d[e], ds[e])[0]

        def fma32(a, b, c):
            return (np.float64(a) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)

        def rows_fn(rows, idx, w, x, logits, norm):
            i_, w_, _ = o.route_topk(logits.numpy(), K)
            idx.copy_(torch.from_numpy(i_)); w.copy_(torch.from_numpy(w_))
            rows.zero_()
            for k, e in enumerate(i_[0].tolist()):
                if lo <= e < hi:
                    rows[k] = torch.from_numpy(expert_row(x.numpy(), e))

        def combine_fn(rows, w, idx, order_):
            acc = np.zeros(D, np.float32)
            for k in range(K):
                acc = fma32(w[0, k].item(), rows[k].numpy(), acc)
            return torch.from_numpy(acc[None])

        def partial_fn(x_all, l_all, order_, norm):
            i_, w_, _ = o.route_topk(l_all.numpy(), K)
            out = np.zeros(x_all.shape, np.float32)
            for t in range(x_all.shape[0]):
                ks = sorted(range(K), key=lambda k: int(i_[t, k])) if order_ == 1 else list(range(K))
                for k in ks:
                    if lo <= i_[t, k] < hi:
                        out[t] = fma32(w_[t, k], expert_row(x_all[t:t + 1].numpy(), int(i_[t, k])), out[t])
            return torch.from_numpy(out)

        ep = ExpertParallelMoe(E, K, I, D, rows_fn=rows_fn, combine_fn=combine_fn, partial_fn=partial_fn)
        rng = np.random.default_rng(6)
        for _ in range(3):                                   # the same token on every rank
            x = rng.standard_normal((1, D)).astype(np.float32); lg = (rng.standard_normal((1, E)) * 0.7).astype(np.float32)
            got = ep.decode(torch.from_numpy(x), torch.from_numpy(lg)).numpy()
            assert got.tobytes() == o.moe_d1(ex, x, lg)[0].tobytes()
        s = 5                                                # tokens per rank
        x_all = rng.standard_normal((world * s, D)).astype(np.float32)
        lg_all = (rng.standard_normal((world * s, E)) * 0.7).astype(np.float32)
        mine = slice(rank * s, (rank + 1) * s)
        got = ep.forward_gathered(torch.from_numpy(x_all[mine]), torch.from_numpy(lg_all[mine]), order=1).numpy()
        want = o.moe_batch(ex, x_all, lg_all)[0][mine]
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_fixed_size_routes_two_ranks():
    mp.spawn(_fixed_size_worker, args=(2, _free_port()), nprocs=2, join=True)


def _bad_plan_worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moty_b200.parallel import ep_exchange
        rows = torch.zeros((3, 4)); eids = torch.zeros(3, dtype=torch.int32)
        counts = torch.tensor([2, 2])                    # 4 planned, 3 present: every rank must refuse
        with pytest.raises(RuntimeError, match="dispatch plan disagrees"):
            ep_exchange(rows, eids, counts)
    finally:
        dist.destroy_process_group()


def test_inconsistent_dispatch_plan_is_refused():
    mp.spawn(_bad_plan_worker, args=(2, _free_port()), nprocs=2, join=True)
