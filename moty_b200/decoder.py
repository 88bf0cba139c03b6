"""A dense decoder step on one GPU, composed from the library's device entries the way the reference's
``qwen`` engine composes its CPU functions (engines/qwen.c:681-740, ``step``): embedding rows, then per
layer RMS norm -> q/k/v projections -> attention core -> o projection -> residual add -> RMS norm ->
SwiGLU FFN -> residual add, then the final norm of the last token, the (tied) lm_head and the greedy
pick.  Activations stay on the device; only token ids go in and one id (or the logits) comes out.

This is host-side glue for tests and for the decode rows of ``bench.py``; the arithmetic is in the C-ABI
entries it calls (``moty_cuda_mat_apply_dev``, ``moty_cuda_attn_core_dev``, ``moty_cuda_ffn_dev``,
``moty_cuda_rmsnorm_dev``, ``moty_cuda_add_dev``, ``moty_cuda_embed_rows_dev``, ``moty_cuda_head_argmax_dev``).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import Attn, Mat, MotyCudaError, lib, stream_handle, ACT_GELU_TANH, ACT_SILU


def _ck(rc):
    if rc != 0:
        raise MotyCudaError(f"libmoty_cuda error {rc}: {lib().moty_cuda_last_error().decode()}")


class DenseLayer:
    """One layer's weights: int8 matrices (q, k, v, o, gate, up, down) and f32 norm gains."""

    def __init__(self, q, k, v, o, gate, up, down, in_ln, post_ln, qn=None, kn=None, qkv=None, moe=None, norm_topk=1):
        self.q, self.k, self.v, self.o, self.gate, self.up, self.down = q, k, v, o, gate, up, down
        self.in_ln, self.post_ln, self.qn, self.kn = in_ln, post_ln, qn, kn
        # optional: the rows of q, k and v in one matrix (the reference's fused [q|k|v], nn/attn.h:24): one product
        # per decode token instead of three; per-row quantization makes the concatenation exact
        self.qkv = qkv
        # optional: a routed layer (moty_b200.Moe with its router set) in place of the dense FFN, combined per token in
        # selection order as engines/olmoe.c:219-244 does; gate/up/down may then be None
        self.moe, self.norm_topk = moe, norm_topk


class DenseDecoder:
    """``layers``: list of DenseLayer (matrices as ``moty_b200.Mat``, gains as numpy f32); ``head``: the lm_head
    ``Mat`` (MOTY_WF_I8 [vocab][D]; with tied embeddings it is also the embedding table); ``final_norm`` [D]."""

    def __init__(self, layers, head: Mat, final_norm, n_heads, n_kv_heads, head_dim, max_t, theta=1e6, eps=1e-6,
                 rot=None, kv8=False, device=0, max_S=64, fold_addnorm=None, fold_ffn=False):
        import torch
        self.torch = torch
        self.dev = torch.device(f"cuda:{device}")
        self.layers, self.head = layers, head
        self.H, self.KV, self.hd, self.eps, self.max_t = n_heads, n_kv_heads, head_dim, float(eps), max_t
        self.D = head.I
        # fold the add+norm in front of a layer's [q|k|v] product into that launch (one token): measured a gain at hidden
        # 1024 (1391 -> 1428 tok/s replayed) and 2048 once every launch of the layer was chained to the next.  The same
        # fold in front of the dense FFN block (fold_ffn) is built and bit-identical but measured a loss (1428 -> 1398):
        # the ~600 CTAs of the gate/up launch each redo the row, where the separate one-CTA launch is nearly free
        self.fold_addnorm = True if fold_addnorm is None else bool(fold_addnorm)
        self.fold_ffn = bool(fold_ffn)
        f = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(self.dev)
        self.final_norm = f(final_norm)
        self.ln = [(f(l.in_ln), f(l.post_ln)) for l in layers]
        self.attn = [Attn(n_heads, n_kv_heads, head_dim, max_t, theta=theta, eps=eps, rot=rot, qn=l.qn, kn=l.kn, kv8=kv8,
                          device=device) for l in layers]
        self.stream = torch.cuda.Stream(device=self.dev)
        self._alloc(max_S)

    def _alloc(self, S):
        t, dev = self.torch, self.dev
        qw, kw = self.H * self.hd, self.KV * self.hd
        e = lambda *shape: t.empty(shape, device=dev, dtype=t.float32)
        self._drop_graph()                       # a captured step holds the addresses of the buffers replaced below
        self.cap = S
        self.x, self.nrm, self.tmp = e(S, self.D), e(S, self.D), e(S, self.D)
        self.x_alt = e(1, self.D)
        self.qb, self.kb, self.vb, self.ctx = e(S, qw), e(S, kw), e(S, kw), e(S, qw)
        self.qkvb = e(1, qw + 2 * kw)
        self.ids = t.empty((S,), device=dev, dtype=t.int32)
        self.out_id = t.empty((1,), device=dev, dtype=t.int32)
        self.logits = e(1, self.head.O)

    def _drop_graph(self):
        """Forget the captured decode step and let the library's scratch grow again."""
        if getattr(self, "_graph", None) is not None:
            self._graph = None
            _ck(lib().moty_cuda_scratch_freeze(self.dev.index or 0, 0))

    def _check_kernels(self):
        """After a stream synchronisation: did a bounded wait inside a kernel run out (incomplete results)?"""
        _ck(lib().moty_cuda_kernel_status(self.dev.index or 0, C.c_void_p(stream_handle(self.stream))))

    def step(self, ids, pos_base, want_logits=False):
        """Tokens ``ids`` at positions pos_base.. : returns the greedy next token after the last of them
        (and the last token's logits when asked)."""
        t, L = self.torch, lib()
        ids = np.ascontiguousarray(ids, np.int32).ravel()
        S = ids.size
        if S > getattr(self, "_max_S", 0):
            self._drop_graph()                   # a larger batch than any before may grow the library's scratch
            self._max_S = S
        if S > self.cap:
            self._alloc(S)
        if pos_base + S > self.max_t:
            raise MotyCudaError(f"positions {pos_base}..{pos_base + S} exceed the cache of {self.max_t}")
        D = self.D
        p = lambda ten: C.c_void_p(ten.data_ptr())
        with t.cuda.stream(self.stream):
            sh = C.c_void_p(stream_handle(self.stream))
            self.ids[:S].copy_(t.from_numpy(ids), non_blocking=True)
            _ck(L.moty_cuda_embed_rows_dev(self.head.h, p(self.x), p(self.ids), S, C.c_float(1.0), sh))
            x = self._layers(S, pos_base, None, sh)
            last = x[S - 1:S]
            _ck(L.moty_cuda_rmsnorm_dev(p(self.nrm), p(last), p(self.final_norm), 1, D, C.c_float(self.eps), sh))
            _ck(L.moty_cuda_head_argmax_dev(self.head.h, p(self.nrm), 1, p(self.out_id), p(self.logits), sh))
            tok = int(self.out_id.cpu()[0])          # waits for the stream
            self._check_kernels()
            if want_logits:
                return tok, self.logits.cpu().numpy()[0]
        return tok

    def _layers(self, S, pos_base, pos_dev, sh):
        """The layers of engines/qwen.c:696-712 on self.x [S][D].  A residual add and the norm that follows it are one
        launch (same results); with S = 1 and a fused matrix the three projections are one product, and the add+norm in
        front of that product and in front of a dense FFN block ride inside those launches (same bits; the sum goes to
        the other of two residual buffers)."""
        L, D, eps = lib(), self.D, C.c_float(self.eps)
        p = lambda ten: C.c_void_p(ten.data_ptr())
        qw, kw = self.H * self.hd, self.KV * self.hd
        nl = len(self.layers)
        x, x_alt = self.x, self.x_alt
        one = self.fold_addnorm and S == 1
        fold_qkv = [one and l.qkv is not None and bool(L.moty_cuda_mat_addnorm_supported(l.qkv.h)) for l in self.layers]
        fold_ffn = [self.fold_ffn and S == 1 and l.moe is None and bool(L.moty_cuda_ffn_resnorm_supported(l.gate.h, l.up.h))
                    for l in self.layers]
        pending = False                          # self.tmp holds a block output that has not been added to x yet
        _ck(L.moty_cuda_rmsnorm_dev(p(self.nrm), p(x), p(self.ln[0][0]), S, D, eps, sh))
        for i, (l, (in_ln, post_ln), a) in enumerate(zip(self.layers, self.ln, self.attn)):
            if S == 1 and l.qkv is not None:
                if pending:
                    _ck(L.moty_cuda_mat_apply_resnorm_dev(l.qkv.h, p(self.qkvb), p(x), p(self.tmp), None, p(x_alt), p(in_ln), eps, sh))
                    x, x_alt = x_alt, x
                    pending = False
                else:
                    _ck(L.moty_cuda_mat_apply_dev(l.qkv.h, p(self.qkvb), p(self.nrm), 1, sh))
                base = self.qkvb.data_ptr()
                qp, kp, vp = C.c_void_p(base), C.c_void_p(base + 4 * qw), C.c_void_p(base + 4 * (qw + kw))
            else:
                _ck(L.moty_cuda_mat_apply_dev(l.q.h, p(self.qb), p(self.nrm), S, sh))
                _ck(L.moty_cuda_mat_apply_dev(l.k.h, p(self.kb), p(self.nrm), S, sh))
                _ck(L.moty_cuda_mat_apply_dev(l.v.h, p(self.vb), p(self.nrm), S, sh))
                qp, kp, vp = p(self.qb), p(self.kb), p(self.vb)
            if pos_dev is None:
                _ck(L.moty_cuda_attn_core_dev(a.h, p(self.ctx), qp, kp, vp, S, pos_base, sh))
            else:
                _ck(L.moty_cuda_attn_core_posdev(a.h, p(self.ctx), qp, kp, vp, S, p(pos_dev), pos_base, sh))
            _ck(L.moty_cuda_mat_apply_dev(l.o.h, p(self.tmp), p(self.ctx), S, sh))
            if fold_ffn[i]:
                _ck(L.moty_cuda_ffn_resnorm_dev(l.gate.h, l.up.h, l.down.h, ACT_SILU, p(self.tmp), p(x), p(self.tmp), None, p(x_alt),
                                                p(post_ln), eps, sh))
                x, x_alt = x_alt, x
            else:
                _ck(L.moty_cuda_add_rmsnorm_dev(p(x), p(self.tmp), p(self.nrm), p(post_ln), S, D, eps, sh))
                if l.moe is not None:
                    _ck(L.moty_cuda_moe_apply_dev(l.moe.h, p(self.tmp), p(self.nrm), S, None, 0, l.norm_topk, None, None, sh))
                else:
                    _ck(L.moty_cuda_ffn_dev(l.gate.h, l.up.h, l.down.h, ACT_SILU, p(self.tmp), p(self.nrm), S, sh))
            if i + 1 < nl and fold_qkv[i + 1]:
                pending = True
            elif i + 1 < nl:
                _ck(L.moty_cuda_add_rmsnorm_dev(p(x), p(self.tmp), p(self.nrm), p(self.ln[i + 1][0]), S, D, eps, sh))
            else:
                _ck(L.moty_cuda_add_dev(p(x), p(self.tmp), C.c_longlong(S * D), sh))
        return x

    def _decode_body(self, sh):
        """One greedy step with everything on the device: the token comes from ``self.ids[0]``, the position from
        ``self.pos_dev``; the new token goes to ``self.ids[0]`` and ``self.hist[self.cnt]``, position and count move on."""
        L, D = lib(), self.D
        p = lambda ten: C.c_void_p(ten.data_ptr())
        _ck(L.moty_cuda_embed_rows_dev(self.head.h, p(self.x), p(self.ids), 1, C.c_float(1.0), sh))
        x = self._layers(1, self.max_t - 1, self.pos_dev, sh)
        _ck(L.moty_cuda_rmsnorm_dev(p(self.nrm), p(x), p(self.final_norm), 1, D, C.c_float(self.eps), sh))
        _ck(L.moty_cuda_head_argmax_dev(self.head.h, p(self.nrm), 1, p(self.out_id), p(self.logits), sh))
        self.ids[:1].copy_(self.out_id)
        self.hist.index_copy_(0, self.cnt, self.out_id)
        self.pos_dev += 1
        self.cnt += 1

    def greedy_graph(self, first_tok, pos0, n):
        """n greedy tokens after ``first_tok`` at position pos0, the decode step captured ONCE into a CUDA graph and
        replayed n times (the attention core reads its position from the device).  Returns the n token ids."""
        t = self.torch
        if pos0 + n > self.max_t:
            raise MotyCudaError(f"positions {pos0}..{pos0 + n} exceed the cache of {self.max_t}")
        if getattr(self, "pos_dev", None) is None:                       # persistent: the captured graph holds their addresses
            self.pos_dev = t.zeros((1,), device=self.dev, dtype=t.int32)
            self.cnt = t.zeros((1,), device=self.dev, dtype=t.int64)
            self.hist = t.zeros((self.max_t + 1,), device=self.dev, dtype=t.int32)

        def reset(tok, pos):
            self.ids[:1].fill_(int(tok)); self.pos_dev.fill_(int(pos)); self.cnt.zero_()

        if getattr(self, "_graph", None) is None:
            with t.cuda.stream(self.stream):                             # one plain run first: scratch buffers, kernel attributes
                reset(first_tok, pos0)
                self._decode_body(C.c_void_p(stream_handle(self.stream)))
            self.stream.synchronize()
            # from here on the library's scratch may not move: the graph holds its addresses
            _ck(lib().moty_cuda_scratch_freeze(self.dev.index or 0, 1))
            g = t.cuda.CUDAGraph()
            with t.cuda.graph(g, stream=self.stream):
                self._decode_body(C.c_void_p(stream_handle(t.cuda.current_stream())))
            self._graph = g
        with t.cuda.stream(self.stream):
            reset(first_tok, pos0)
            for _ in range(n):
                self._graph.replay()
        self.stream.synchronize()
        self._check_kernels()
        return [int(v) for v in self.hist[:n].cpu().numpy()]

    def close(self):
        self._drop_graph()                       # lifts the scratch freeze taken for the captured step
        for a in self.attn:
            a.close()

    def __del__(self):
        try:
            self._drop_graph()
        except Exception:
            pass


class GemmaLayer:
    """One layer of the reference's ``gemma`` engine (engines/gemma.c:299-386, :392-401, :466-483): int8 matrices
    (q, k, v, o, gate, up, down; optionally the rows of q, k and v in one matrix), the four sandwich norms and the three
    per-head norms as MULTIPLIERS (1 + w for a zero-centred checkpoint), and the layer's own attention geometry: a
    sliding layer has ``window`` > 0 and rotates every pair (``rot`` = head_dim / 2); a global one has ``window`` = 0,
    its own head_dim / KV-head count / theta, and ``rot`` rotated pairs of the p-RoPE."""

    def __init__(self, q, k, v, o, gate, up, down, in_ln, post_attn_ln, pre_ff_ln, post_ff_ln, qn, kn, vn=None, *, n_kv_heads, head_dim,
                 theta, window=0, rot=None, scale=0.0, qkv=None):
        self.q, self.k, self.v, self.o, self.gate, self.up, self.down, self.qkv = q, k, v, o, gate, up, down, qkv
        self.in_ln, self.post_attn_ln, self.pre_ff_ln, self.post_ff_ln = in_ln, post_attn_ln, pre_ff_ln, post_ff_ln
        self.qn, self.kn, self.vn = qn, kn, vn
        self.KV, self.hd, self.theta, self.window, self.scale = n_kv_heads, head_dim, float(theta), int(window), float(scale)
        self.rot = head_dim // 2 if rot is None else int(rot)


class GemmaDecoder(DenseDecoder):
    """The step of engines/gemma.c:453-497 without the per-layer-embedding branch (ple_dim = 0) and without shared KV
    layers: embedding rows scaled by sqrt(hidden), per layer  x += post_attn_norm(attn(in_norm(x)))  and
    x += post_ff_norm(gelu_mlp(pre_ff_norm(x))), the final norm of the last token, the lm_head and the greedy pick.
    The final logit soft-cap (softcap * tanhf(logit / softcap)) is monotonic, so the greedy pick is taken from the
    uncapped logits; ``step(..., want_logits=True)`` returns them uncapped."""

    def __init__(self, layers, head: Mat, final_norm, n_heads, max_t, eps=1e-6, kv8=False, device=0, max_S=64, fold_addnorm=False,
                 fold_ffn=False):
        # the folds of the sandwich steps into their consumers are built and bit-identical, and off by default: at hidden
        # 3840 they measured a loss (289 -> 263 tok/s replayed on the 48-layer shape; every CTA of the consumer redoes two
        # reductions over the row, where the separate one-CTA launch is nearly free under programmatic dependent launch)
        import torch
        self.torch = torch
        self.dev = torch.device(f"cuda:{device}")
        self.layers, self.head = layers, head
        self.H, self.eps, self.max_t = n_heads, float(eps), max_t
        self.D = head.I
        self.embed_scale = float(np.sqrt(np.float32(self.D)))
        self.fold_addnorm, self.fold_ffn = bool(fold_addnorm), bool(fold_ffn)
        f = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(self.dev)
        self.final_norm = f(final_norm)
        self.ln = [tuple(f(g) for g in (l.in_ln, l.post_attn_ln, l.pre_ff_ln, l.post_ff_ln)) for l in layers]
        self.attn = [Attn(n_heads, l.KV, l.hd, max_t, theta=l.theta, eps=eps, rot=l.rot, qn=l.qn, kn=l.kn, vn=l.vn, kv8=kv8,
                          device=device, gemma=True, window=l.window, scale=l.scale) for l in layers]
        # buffers sized for the widest layer
        self.hd, self.KV = max(l.hd for l in layers), 0
        self._qw = max(n_heads * l.hd for l in layers)
        self._kw = max(l.KV * l.hd for l in layers)
        self.stream = torch.cuda.Stream(device=self.dev)
        self._alloc(max_S)

    def _alloc(self, S):
        t, dev = self.torch, self.dev
        e = lambda *shape: t.empty(shape, device=dev, dtype=t.float32)
        self._drop_graph()
        self.cap = S
        self.x, self.nrm, self.tmp = e(S, self.D), e(S, self.D), e(S, self.D)
        self.x_alt = e(1, self.D)
        self.qb, self.kb, self.vb, self.ctx = e(S, self._qw), e(S, self._kw), e(S, self._kw), e(S, self._qw)
        self.qkvb = e(1, self._qw + 2 * self._kw)
        self.ids = t.empty((S,), device=dev, dtype=t.int32)
        self.out_id = t.empty((1,), device=dev, dtype=t.int32)
        self.logits = e(1, self.head.O)

    def _embed(self, S, sh):
        p = lambda ten: C.c_void_p(ten.data_ptr())
        _ck(lib().moty_cuda_embed_rows_dev(self.head.h, p(self.x), p(self.ids), S, C.c_float(self.embed_scale), sh))

    def _layers(self, S, pos_base, pos_dev, sh):
        """engines/gemma.c:466-483 on self.x [S][D]; on return self.nrm holds the FINAL norm of every row (the last
        sandwich step opens it), so the caller goes straight to the lm_head.  With one token the sandwich steps in front
        of the fused [q|k|v] product and in front of the FFN block ride inside those launches (same bits)."""
        L, D, eps = lib(), self.D, C.c_float(self.eps)
        p = lambda ten: C.c_void_p(ten.data_ptr())
        nl = len(self.layers)
        x, x_alt = self.x, self.x_alt
        one = self.fold_addnorm and S == 1
        fold_qkv = [one and l.qkv is not None and bool(L.moty_cuda_mat_addnorm_supported(l.qkv.h)) for l in self.layers]
        fold_ffn = [self.fold_ffn and S == 1 and bool(L.moty_cuda_ffn_resnorm_supported(l.gate.h, l.up.h)) for l in self.layers]
        pending = None                           # gains of the post-FFN norm whose sandwich step is still owed (t in self.tmp)
        _ck(L.moty_cuda_rmsnorm_dev(p(self.nrm), p(x), p(self.ln[0][0]), S, D, eps, sh))
        for i, (l, (in_ln, post_attn, pre_ff, post_ff), a) in enumerate(zip(self.layers, self.ln, self.attn)):
            qw, kw = self.H * l.hd, l.KV * l.hd
            if S == 1 and l.qkv is not None:
                if pending is not None:
                    _ck(L.moty_cuda_mat_apply_resnorm_dev(l.qkv.h, p(self.qkvb), p(x), p(self.tmp), p(pending), p(x_alt), p(in_ln), eps, sh))
                    x, x_alt = x_alt, x
                    pending = None
                else:
                    _ck(L.moty_cuda_mat_apply_dev(l.qkv.h, p(self.qkvb), p(self.nrm), 1, sh))
                base = self.qkvb.data_ptr()
                qp, kp, vp = C.c_void_p(base), C.c_void_p(base + 4 * qw), C.c_void_p(base + 4 * (qw + kw))
            else:
                _ck(L.moty_cuda_mat_apply_dev(l.q.h, p(self.qb), p(self.nrm), S, sh))
                _ck(L.moty_cuda_mat_apply_dev(l.k.h, p(self.kb), p(self.nrm), S, sh))
                _ck(L.moty_cuda_mat_apply_dev(l.v.h, p(self.vb), p(self.nrm), S, sh))
                qp, kp, vp = p(self.qb), p(self.kb), p(self.vb)
            if pos_dev is None:
                _ck(L.moty_cuda_attn_core_dev(a.h, p(self.ctx), qp, kp, vp, S, pos_base, sh))
            else:
                _ck(L.moty_cuda_attn_core_posdev(a.h, p(self.ctx), qp, kp, vp, S, p(pos_dev), pos_base, sh))
            _ck(L.moty_cuda_mat_apply_dev(l.o.h, p(self.tmp), p(self.ctx), S, sh))
            if fold_ffn[i]:
                _ck(L.moty_cuda_ffn_resnorm_dev(l.gate.h, l.up.h, l.down.h, ACT_GELU_TANH, p(self.tmp), p(x), p(self.tmp), p(post_attn),
                                                p(x_alt), p(pre_ff), eps, sh))
                x, x_alt = x_alt, x
            else:
                _ck(L.moty_cuda_normadd_rmsnorm_dev(p(x), p(self.tmp), p(post_attn), p(self.nrm), p(pre_ff), S, D, eps, sh))
                _ck(L.moty_cuda_ffn_dev(l.gate.h, l.up.h, l.down.h, ACT_GELU_TANH, p(self.tmp), p(self.nrm), S, sh))
            if i + 1 < nl and fold_qkv[i + 1]:
                pending = post_ff
            else:
                nxt = self.ln[i + 1][0] if i + 1 < nl else self.final_norm
                _ck(L.moty_cuda_normadd_rmsnorm_dev(p(x), p(self.tmp), p(post_ff), p(self.nrm), p(nxt), S, D, eps, sh))
        return x

    def step(self, ids, pos_base, want_logits=False):
        t, L = self.torch, lib()
        ids = np.ascontiguousarray(ids, np.int32).ravel()
        S = ids.size
        if S > getattr(self, "_max_S", 0):
            self._drop_graph()
            self._max_S = S
        if S > self.cap:
            self._alloc(S)
        if pos_base + S > self.max_t:
            raise MotyCudaError(f"positions {pos_base}..{pos_base + S} exceed the cache of {self.max_t}")
        p = lambda ten: C.c_void_p(ten.data_ptr())
        with t.cuda.stream(self.stream):
            sh = C.c_void_p(stream_handle(self.stream))
            self.ids[:S].copy_(t.from_numpy(ids), non_blocking=True)
            self._embed(S, sh)
            self._layers(S, pos_base, None, sh)
            _ck(L.moty_cuda_head_argmax_dev(self.head.h, p(self.nrm[S - 1:S]), 1, p(self.out_id), p(self.logits), sh))
            tok = int(self.out_id.cpu()[0])
            self._check_kernels()
            if want_logits:
                return tok, self.logits.cpu().numpy()[0]
        return tok

    def prefill(self, ids, pos_base=0, block=512):
        """A long prompt in blocks of ``block`` tokens (the blocked prefill of engines/gemma.c:484-485: the blocks
        before the last need no logits); returns the greedy token after the last one."""
        ids = np.ascontiguousarray(ids, np.int32).ravel()
        tok = None
        for lo in range(0, ids.size, block):
            tok = self.step(ids[lo:lo + block], pos_base + lo)
        return tok

    def _decode_body(self, sh):
        L = lib()
        p = lambda ten: C.c_void_p(ten.data_ptr())
        self._embed(1, sh)
        self._layers(1, self.max_t - 1, self.pos_dev, sh)
        _ck(L.moty_cuda_head_argmax_dev(self.head.h, p(self.nrm), 1, p(self.out_id), p(self.logits), sh))
        self.ids[:1].copy_(self.out_id)
        self.hist.index_copy_(0, self.cnt, self.out_id)
        self.pos_dev += 1
        self.cnt += 1
