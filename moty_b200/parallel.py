"""Sharding of the quantized-matmul path over the GPUs of one box.

One process per GPU; ``torch.distributed`` (NCCL over NVLink on GPUs, gloo on
CPU for the host-logic tests) is the plumbing.  The reference is a single
process, so nothing here has a reference counterpart; the parity statement is
"the sharded result equals the one-GPU result":

* ``RowShardedMat``     rows of a matrix split over the ranks, all-gather of the
                        output slices.  Every output element is computed whole on
                        one GPU, so the gathered result is bit-identical.
* ``ExpertParallelMoe`` experts split over the ranks in contiguous id ranges.  Three routes:
    ``decode``          one token replicated on every rank (its hidden state is, when the
                        attention is replicated): every rank routes it redundantly and runs its
                        resident experts in the one-launch decode kernel, which also leaves each
                        selected expert's own output row in a [K][D] table (zeros for experts of
                        other ranks).  ONE fixed-size all-reduce of that table (x + 0 is exact)
                        and the combine in selection order: the one-GPU bits, no count exchange,
                        no host synchronisation.
    ``decode_peer``     the same with the exchange done by the library's own kernels over NVLink peer
                        memory: the decode kernel stores the rows of its experts straight into every rank's
                        row table; the next launch signals the peers (fence + release store per peer), waits
                        -- bounded -- for their rows and combines.  No collective; the one-GPU bits.
    ``forward_gathered``  prefill: all-gather of the ranks' token shards and logits (with K = 8
                        selections per token and 8 ranks this moves the bytes a dispatch of routed
                        copies would), every rank routes all tokens redundantly and computes the
                        partial sums of its experts, one reduce-scatter returns each rank its own
                        tokens.  Two fixed-size collectives, no host synchronisation; the sum
                        over ranks is taken in the collective's order, so the result agrees with
                        the one-GPU block to f32 rounding (1e-5), not bit for bit.
    ``forward``         the exact route: routed rows travel to the expert's owner and the
                        expert outputs travel back (all-to-all both ways, sizes planned on the
                        host); the home rank combines them in the reference's order:
                        bit-identical to the one-GPU block.

No kernel here waits on another rank: every exchange is a stream-ordered
collective of the communication library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import WF_I8, Mat, Moe, _ck, lib, stream_handle


def shard_rows(O: int, world: int, rank: int, align: int = 1):
    """Contiguous row range of `rank`: equal shards of ceil(O / world) rounded up
    to `align` rows (4 for Q4R4 blocks); the last ranks may get fewer or none."""
    per = -(-O // world)
    per = -(-per // align) * align
    lo = min(rank * per, O)
    return lo, min(lo + per, O), per


def shard_experts(E: int, world: int, rank: int):
    """Contiguous expert range of `rank` (E divisible by world, as in the configs: 64/32/16/8 per GPU)."""
    if E % world:
        raise ValueError(f"{E} experts do not split evenly over {world} ranks")
    per = E // world
    return rank * per, (rank + 1) * per


# ---------------------------------------------------------------------------
# row-sharded dense matrix
# ---------------------------------------------------------------------------
class RowShardedMat:
    """Rows [lo, hi) of a matrix on this rank; ``apply`` returns the full [S][O]."""

    def __init__(self, fmt, codes, scales, O, I, device=0, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.O, self.I = O, I
        align = 4 if fmt != WF_I8 else 1
        self.lo, self.hi, self.per = shard_rows(O, self.world, self.rank, align)
        self.mat = Mat(fmt, codes, scales, O, I, device, rows=(self.lo, self.hi)) if self.hi > self.lo else None
        self.dev = torch.device("cuda", device)

    @classmethod
    def from_local_rows(cls, fmt, codes_local, scales_local, O, I, device=0, group=None):
        """The same shard built from this rank's rows only (a loader that reads just its slice of a big matrix):
        codes_local / scales_local hold rows [lo, hi) of the O x I matrix, lo/hi from shard_rows."""
        self = cls.__new__(cls)
        self.group = group
        self.world = dist.get_world_size(group); self.rank = dist.get_rank(group)
        self.O, self.I = O, I
        self.lo, self.hi, self.per = shard_rows(O, self.world, self.rank, 4 if fmt != WF_I8 else 1)
        self.mat = Mat(fmt, codes_local, scales_local, self.hi - self.lo, I, device) if self.hi > self.lo else None
        self.dev = torch.device("cuda", device)
        return self

    def apply(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        """x [S][I] f32 on this GPU (replicated on every rank) -> y [S][O] on every rank."""
        S = x.shape[0]
        st = stream or torch.cuda.current_stream(self.dev)
        part = torch.zeros((S, self.per), dtype=torch.float32, device=self.dev)
        if self.mat is not None:
            n = self.hi - self.lo
            if n == self.per:
                from . import mat_apply_dev
                mat_apply_dev(self.mat, part.data_ptr(), x.data_ptr(), S, stream_handle(st))
            else:                                   # ragged last shard: compute compact, copy into the padded slot
                from . import mat_apply_dev
                tmp = torch.empty((S, n), dtype=torch.float32, device=self.dev)
                mat_apply_dev(self.mat, tmp.data_ptr(), x.data_ptr(), S, stream_handle(st))
                part[:, :n] = tmp
        gathered = torch.empty((self.world, S, self.per), dtype=torch.float32, device=self.dev)
        dist.all_gather_into_tensor(gathered, part, group=self.group)
        return gathered.permute(1, 0, 2).reshape(S, self.world * self.per)[:, : self.O].contiguous()

    def decode(self, x: torch.Tensor, stream=None) -> torch.Tensor:
        """One row, x [1][I] replicated -> y [1][world * per] (the first O entries are the product).  The rank's slice is
        written straight into its slot of a buffer kept across calls, one all-gather in place, nothing else."""
        st = stream or torch.cuda.current_stream(self.dev)
        if getattr(self, "_dec", None) is None:
            self._dec = torch.zeros((self.world, self.per), dtype=torch.float32, device=self.dev)
        if self.mat is not None:
            from . import mat_apply_dev
            mat_apply_dev(self.mat, self._dec[self.rank].data_ptr(), x.data_ptr(), 1, stream_handle(st))
        dist.all_gather_into_tensor(self._dec, self._dec[self.rank], group=self.group)
        return self._dec.view(1, self.world * self.per)


# ---------------------------------------------------------------------------
# expert-parallel exchange plan (pure tensor logic: runs on CPU tensors too)
# ---------------------------------------------------------------------------
def ep_dispatch_plan(idx: torch.Tensor, experts_per_rank: int, world: int):
    """idx [s][K] expert ids of this rank's tokens.  Returns
    order   [s*K]  positions of the selections sorted by owner rank (stable: token-major inside a rank)
    counts  [world] selections per owner rank."""
    owner = (idx.reshape(-1) // experts_per_rank).to(torch.int64)
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=world)
    return order, counts


def ep_exchange(rows: torch.Tensor, eids: torch.Tensor, counts: torch.Tensor, group=None):
    """All-to-all of routed rows [P][D] (already in owner order) and their expert ids.
    Returns (recv_rows, recv_eids, recv_counts)."""
    world = dist.get_world_size(group)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)
    send = [int(v) for v in counts.tolist()]
    recv = [int(v) for v in recv_counts.tolist()]
    if sum(send) != rows.shape[0]:
        raise RuntimeError(f"dispatch plan disagrees with its rows: {sum(send)} planned, {rows.shape[0]} present")
    recv_rows = torch.empty((sum(recv), rows.shape[1]), dtype=rows.dtype, device=rows.device)
    recv_eids = torch.empty((sum(recv),), dtype=eids.dtype, device=eids.device)
    dist.all_to_all_single(recv_rows, rows.contiguous(), recv, send, group=group)
    dist.all_to_all_single(recv_eids, eids.contiguous(), recv, send, group=group)
    return recv_rows, recv_eids, recv_counts


def ep_return(h: torch.Tensor, counts: torch.Tensor, recv_counts: torch.Tensor, group=None):
    """The way back: expert outputs [sum(recv)][D] to the ranks that sent the rows."""
    send = [int(v) for v in recv_counts.tolist()]
    recv = [int(v) for v in counts.tolist()]
    back = torch.empty((sum(recv), h.shape[1]), dtype=h.dtype, device=h.device)
    dist.all_to_all_single(back, h.contiguous(), recv, send, group=group)
    return back


class ExpertParallelMoe:
    """One MoE layer with its experts spread over the ranks (contiguous id ranges)
    and the tokens sharded over the ranks.  ``forward`` takes this rank's tokens
    and router logits and returns this rank's outputs.

    expert_fn / combine_fn / route_fn default to the CUDA library; the CPU tests of
    the exchange logic pass numpy stand-ins."""

    def __init__(self, E, K, I, D, efmt=WF_I8, device=0, group=None, moe: Moe | None = None,
                 expert_fn=None, combine_fn=None, route_fn=None, rows_fn=None, partial_fn=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.E, self.K, self.I, self.D = E, K, I, D
        self.e_lo, self.e_hi = shard_experts(E, self.world, self.rank)
        self.per = E // self.world
        self.moe = moe
        self.rows_fn, self.partial_fn = rows_fn, partial_fn
        if moe is None and expert_fn is None and rows_fn is None and partial_fn is None:
            self.moe = Moe(E, K, I, D, efmt, self.e_lo, self.e_hi, device)
        self.expert_fn, self.combine_fn, self.route_fn = expert_fn, combine_fn, route_fn

    def upload_expert(self, eid, g, gs, u, us, d, ds):
        if self.e_lo <= eid < self.e_hi:
            self.moe.upload_expert(eid, g, gs, u, us, d, ds)

    # -- the three compute steps (CUDA library by default) ------------------
    def _route(self, logits, norm_topk):
        if self.route_fn is not None:
            return self.route_fn(logits, self.K, norm_topk)
        s = logits.shape[0]
        idx = torch.empty((s, self.K), dtype=torch.int32, device=logits.device)
        w = torch.empty((s, self.K), dtype=torch.float32, device=logits.device)
        st = stream_handle(torch.cuda.current_stream(logits.device))
        _ck(lib().moty_cuda_route_topk_dev(C.c_void_p(logits.data_ptr()), s, self.E, self.K, C.c_void_p(idx.data_ptr()),
                                           C.c_void_p(w.data_ptr()), None, int(norm_topk), C.c_void_p(st)))
        return idx, w

    def _experts(self, rows, eids):
        if self.expert_fn is not None:
            return self.expert_fn(rows, eids)
        h = torch.empty_like(rows)
        if rows.shape[0]:
            st = stream_handle(torch.cuda.current_stream(rows.device))
            _ck(lib().moty_cuda_moe_experts_dev(self.moe.h, C.c_void_p(h.data_ptr()), C.c_void_p(rows.data_ptr()),
                                                C.c_void_p(eids.data_ptr()), rows.shape[0], C.c_void_p(st)))
        return h

    def _combine(self, h_sk, w, idx, order):
        if self.combine_fn is not None:
            return self.combine_fn(h_sk, w, idx, order)
        s = w.shape[0]
        out = torch.empty((s, self.D), dtype=torch.float32, device=h_sk.device)
        if s:
            st = stream_handle(torch.cuda.current_stream(h_sk.device))
            _ck(lib().moty_cuda_moe_combine_dev(C.c_void_p(out.data_ptr()), C.c_void_p(h_sk.data_ptr()),
                                                C.c_void_p(w.data_ptr()), C.c_void_p(idx.data_ptr()),
                                                s, self.K, self.D, int(order), C.c_void_p(st)))
        return out

    def decode(self, x: torch.Tensor, logits: torch.Tensor, norm_topk: int = 1) -> torch.Tensor:
        """One token replicated on every rank: x [1][D], logits [1][E] -> out [1][D], the one-GPU bits."""
        dev = x.device
        if getattr(self, "_drows", None) is None:
            self._drows = torch.empty((self.K, self.D), dtype=torch.float32, device=dev)
            self._dpart = torch.empty((1, self.D), dtype=torch.float32, device=dev)
            self._didx = torch.empty((1, self.K), dtype=torch.int32, device=dev)
            self._dw = torch.empty((1, self.K), dtype=torch.float32, device=dev)
            self._dout = torch.empty((1, self.D), dtype=torch.float32, device=dev)
        st = stream_handle(torch.cuda.current_stream(dev)) if dev.type == "cuda" else 0
        if self.rows_fn is not None:
            self.rows_fn(self._drows, self._didx, self._dw, x, logits, norm_topk)
        else:
            _ck(lib().moty_cuda_moe_d1_rows_dev(self.moe.h, C.c_void_p(self._drows.data_ptr()), C.c_void_p(self._dpart.data_ptr()),
                                                C.c_void_p(x.data_ptr()), C.c_void_p(logits.data_ptr()), int(norm_topk),
                                                C.c_void_p(self._didx.data_ptr()), C.c_void_p(self._dw.data_ptr()), C.c_void_p(st)))
        dist.all_reduce(self._drows, group=self.group)              # disjoint non-zero rows: the sum is exact
        if self.combine_fn is not None:
            return self.combine_fn(self._drows, self._dw, self._didx, 0)
        _ck(lib().moty_cuda_moe_combine_dev(C.c_void_p(self._dout.data_ptr()), C.c_void_p(self._drows.data_ptr()),
                                            C.c_void_p(self._dw.data_ptr()), C.c_void_p(self._didx.data_ptr()),
                                            1, self.K, self.D, 0, C.c_void_p(st)))
        return self._dout

    def _peer_setup(self, dev):
        """Row tables (two, used alternately) and flag words of every rank in memory all GPUs of the group can address:
        torch's symmetric memory does the allocation and the handle exchange; the kernels only see raw pointers."""
        n_tab = 2 * self.K * self.D
        if self.world == 1:
            buf = torch.zeros((n_tab + 64,), dtype=torch.float32, device=dev)
            ptrs = [buf.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm
            group = self.group or dist.group.WORLD
            try:
                symm.enable_symm_mem_for_group(group.group_name)
            except Exception:
                pass                                             # newer versions enable it at rendezvous
            buf = symm.empty((n_tab + 64,), dtype=torch.float32, device=dev)
            buf.zero_()
            hdl = symm.rendezvous(buf, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            self._peer_hdl = hdl
        torch.cuda.synchronize(dev)
        if self.world > 1:
            dist.barrier(group=self.group)                       # every rank's flags are zero before anyone signals
        self._peer_buf = buf
        self._peer_tables = (C.c_void_p * self.world)(*ptrs)
        self._peer_flags = (C.c_void_p * self.world)(*[p + 4 * n_tab for p in ptrs])
        self._peer_epoch = 0
        self._peer_out = torch.empty((1, self.D), dtype=torch.float32, device=dev)

    def decode_peer(self, x: torch.Tensor, logits: torch.Tensor, norm_topk: int = 1) -> torch.Tensor:
        """``decode`` with the exchange done by the library's own kernels over NVLink peer memory: the decode kernel
        stores its experts' rows into every rank's table, a second launch signals the peers, waits (bounded) for
        theirs and combines.  Two launches per layer, no collective, the one-GPU bits.  Every rank must call it the
        same number of times (the step counter is part of the protocol)."""
        if getattr(self, "_peer_buf", None) is None:
            self._peer_setup(x.device)
        self._peer_epoch += 1
        st = stream_handle(torch.cuda.current_stream(x.device))
        _ck(lib().moty_cuda_moe_d1_peer_dev(self.moe.h, C.c_void_p(self._peer_out.data_ptr()), C.c_void_p(x.data_ptr()),
                                            C.c_void_p(logits.data_ptr()), int(norm_topk), self._peer_tables, self._peer_flags,
                                            self.world, self.rank, C.c_uint(self._peer_epoch), C.c_void_p(st)))
        return self._peer_out

    def forward_gathered(self, x: torch.Tensor, logits: torch.Tensor, order: int = 1, norm_topk: int = 1) -> torch.Tensor:
        """x [s][D], logits [s][E]: this rank's tokens, the same s on every rank -> out [s][D] (1e-5, see the module text)."""
        s = x.shape[0]
        x_all = torch.empty((self.world * s, self.D), dtype=torch.float32, device=x.device)
        l_all = torch.empty((self.world * s, self.E), dtype=torch.float32, device=x.device)
        dist.all_gather_into_tensor(x_all, x.contiguous(), group=self.group)
        dist.all_gather_into_tensor(l_all, logits.contiguous(), group=self.group)
        if self.partial_fn is not None:
            part = self.partial_fn(x_all, l_all, order, norm_topk)
        else:
            part = torch.empty_like(x_all)
            self.moe.apply_dev(part.data_ptr(), x_all.data_ptr(), self.world * s, l_all.data_ptr(), order, norm_topk, 0, 0,
                               stream_handle(torch.cuda.current_stream(x.device)))
        out = torch.empty((s, self.D), dtype=torch.float32, device=x.device)
        if dist.get_backend(self.group) == "gloo":                  # the CPU tests: gloo has no reduce-scatter
            dist.all_reduce(part, group=self.group)
            out.copy_(part[self.rank * s:(self.rank + 1) * s])
        else:
            dist.reduce_scatter_tensor(out, part, group=self.group)
        return out

    def forward(self, x: torch.Tensor, logits: torch.Tensor, order: int = 1, norm_topk: int = 1) -> torch.Tensor:
        """x [s][D], logits [s][E] of this rank's tokens -> out [s][D].  order: 0 = selection
        order (decode / OLMoE), 1 = ascending expert id (the batch path)."""
        s = x.shape[0]
        idx, w = self._route(logits.contiguous(), norm_topk)
        order_sel, counts = ep_dispatch_plan(idx, self.per, self.world)
        tok = (order_sel // self.K)
        rows = x.index_select(0, tok)                            # routed copies of the tokens, owner order
        eids = idx.reshape(-1).index_select(0, order_sel).to(torch.int32)
        recv_rows, recv_eids, recv_counts = ep_exchange(rows, eids, counts, self.group)
        h = self._experts(recv_rows, recv_eids)
        back = ep_return(h, counts, recv_counts, self.group)     # [s*K][D] in owner order
        h_sk = torch.empty_like(back)
        h_sk.index_copy_(0, order_sel, back)                     # undo the permutation: row s*K+k
        return self._combine(h_sk, w, idx, order)
