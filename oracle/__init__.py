"""CPU checkers for the moty quantized-matmul path.  TEST INFRASTRUCTURE ONLY.

Two shared libraries are wrapped here with ctypes + numpy:

* ``Oracle``  -- ``libmoty_oracle.so``, the plain-C restatement (moty_oracle.c);
* ``Ref``     -- ``_ref/libmoty_ref_<tier>.so``, the unmodified reference sources
  compiled by ``oracle/Makefile`` (present only where they were built or shipped
  prebuilt).

Nothing in the shipped package may import this module; it exists for the tests,
the smoke check and the benchmark's CPU-baseline arm.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

WF_F32, WF_I8, WF_I4, WF_I2, WF_I4G, WF_Q4K, WF_Q6K, WF_Q4R4, WF_Q8R4 = range(9)


def _p(a, t=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "array must be contiguous"
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def ref_src_dir() -> str:
    """Where the reference's c/ directory is looked for: $MOTY_REF_SRC, else the make recipe's default."""
    return os.environ.get("MOTY_REF_SRC", "")


def build(ref_src: str | None = None) -> None:
    """Compile the restatement (always) and the reference (when its sources exist)."""
    ref_src = ref_src or ref_src_dir()
    cmd = ["make", "-s", "-C", HERE, "all"] + ([f"REF={ref_src}"] if ref_src else [])
    subprocess.check_call(cmd)


def _cpu_has(flag: str) -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return flag in line.split()
    except OSError:
        pass
    return False


class _ExpertsI8(C.Structure):
    _fields_ = [("E", C.c_int), ("K", C.c_int), ("I", C.c_int), ("D", C.c_int),
                ("g", C.c_void_p), ("u", C.c_void_p), ("d", C.c_void_p),
                ("gs", C.c_void_p), ("us", C.c_void_p), ("ds", C.c_void_p)]


def unpack_i4_rows(q4, n):
    """Per-row int4 rows [..., (n+1)/2] (element 2j in the low nibble, 2j+1 in the high one; hw/hw_scalar.h:14-22) as the
    signed codes nibble - 8 in int8 [..., n]: the integer dots over them are the reference's dot_i4i8 / dot_i4i8p sums."""
    q4 = np.ascontiguousarray(q4, np.uint8)
    out = np.empty(q4.shape[:-1] + (q4.shape[-1] * 2,), np.int8)
    out[..., 0::2] = (q4 & 15).astype(np.int16) - 8
    out[..., 1::2] = (q4 >> 4).astype(np.int16) - 8
    return np.ascontiguousarray(out[..., :n])


class Experts:
    """Expert-major arrays of one MoE layer (int8 per-row or Q4R4)."""

    def __init__(self, E, K, I, D, g, u, d, gs, us, ds):
        self.E, self.K, self.I, self.D = E, K, I, D
        self.g, self.u, self.d, self.gs, self.us, self.ds = (np.ascontiguousarray(a) for a in (g, u, d, gs, us, ds))
        self.c = _ExpertsI8(E, K, I, D, *(a.ctypes.data for a in (self.g, self.u, self.d, self.gs, self.us, self.ds)))


class AttnCache:
    """Host-side KV storage of one layer for the CPU checkers: f32 K, V [KV][max_t][hd], or int8 rows with one scale
    per (head, position) (K8, V8, Ks, Vs), plus the layer's attention parameters."""

    def __init__(self, H, KV, hd, max_t, theta=1e6, eps=1e-6, rot=None, qn=None, kn=None, kv8=False,
                 gemma=False, window=0, scale=0.0, vn=None):
        """gemma=True: engines/gemma.c's attention -- qn/kn/vn are the RAW norm weights w (the multipliers are 1 + w),
        rot = rotated pairs of the p-RoPE, window > 0 = a sliding layer, scale > 0 overrides 1/sqrt(hd)."""
        self.H, self.KV, self.hd, self.max_t = H, KV, hd, max_t
        self.theta, self.eps, self.rot, self.kv8 = float(theta), float(eps), hd if rot is None else rot, bool(kv8)
        self.gemma, self.window, self.scale = bool(gemma), int(window), float(scale)
        self.vn = None if vn is None else _f32(vn)
        self.qn = None if qn is None else _f32(qn); self.kn = None if kn is None else _f32(kn)
        if kv8:
            self.K8 = np.zeros((KV, max_t, hd), np.int8); self.V8 = np.zeros((KV, max_t, hd), np.int8)
            self.Ks = np.zeros((KV, max_t), np.float32); self.Vs = np.zeros((KV, max_t), np.float32)
        else:
            self.K = np.zeros((KV, max_t, hd), np.float32); self.V = np.zeros((KV, max_t, hd), np.float32)


class Oracle:
    """The C restatement.  Shapes follow the reference: x [S][I], y [S][O]."""

    def __init__(self):
        path = os.path.join(HERE, "libmoty_oracle.so")
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        L = self.lib
        L.oracle_qrow_i8.restype = C.c_float
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_dot_i8i8.restype = C.c_int32
        L.oracle_dot_i4i8.restype = C.c_int32
        L.oracle_argmax.restype = C.c_int
        L.oracle_expf.restype = C.c_float
        L.oracle_expf.argtypes = [C.c_float]
        L.oracle_expf_mismatches.restype = C.c_int64
        L.oracle_expf_mismatches.argtypes = [C.c_uint32, C.c_uint32, C.c_int64]
        L.oracle_exp2_tab_entry.restype = C.c_uint64
        L.oracle_exp2_tab_entry.argtypes = [C.c_int]

    # -- scalars -------------------------------------------------------
    def expf(self, x):
        return np.float32(self.lib.oracle_expf(float(np.float32(x))))

    def expf_mismatches(self, first, stride, count):
        """Inputs (as float bit patterns first, first+stride, ...) on which the restated expf and the host's differ."""
        return int(self.lib.oracle_expf_mismatches(int(first), int(stride), int(count)))

    def f16_to_f32(self, h):
        return self.lib.oracle_f16_to_f32(int(h))

    def f32_to_f16(self, f):
        return self.lib.oracle_f32_to_f16(float(np.float32(f)))

    # -- quantizers ----------------------------------------------------
    def qrow_i8(self, x):
        x = _f32(x)
        q = np.empty(x.shape, np.int8)
        s = self.lib.oracle_qrow_i8(_p(x), _p(q), C.c_int(x.size))
        return q, np.float32(s)

    def qrows_i8(self, x):
        x = _f32(x)
        q = np.empty(x.shape, np.int8)
        s = np.empty(x.shape[0], np.float32)
        for r in range(x.shape[0]):
            s[r] = self.lib.oracle_qrow_i8(_p(x[r]), _p(q[r]), C.c_int(x.shape[1]))
        return q, s

    def quant_g32(self, x):
        x = _f32(x)
        I = x.shape[-1]
        rows = x.reshape(-1, I)
        xq = np.empty(rows.shape, np.int8)
        xs = np.empty((rows.shape[0], I // 32), np.float32)
        xsum = np.empty((rows.shape[0], I // 32), np.int32)
        for r in range(rows.shape[0]):
            self.lib.oracle_quant_g32(_p(rows[r]), C.c_int(I), _p(xq[r]), _p(xs[r]), _p(xsum[r]))
        return xq, xs, xsum

    # -- dots and drivers ----------------------------------------------
    def dot_i8i8(self, w, x):
        w = np.ascontiguousarray(w, np.int8); x = np.ascontiguousarray(x, np.int8)
        return int(self.lib.oracle_dot_i8i8(_p(w), _p(x), C.c_int(w.size)))

    def dot_i4i8(self, w4, x):
        w4 = np.ascontiguousarray(w4, np.uint8); x = np.ascontiguousarray(x, np.int8)
        return int(self.lib.oracle_dot_i4i8(_p(w4), _p(x), C.c_int(x.size)))

    def matmul_q_s(self, x, q, scale, want_acc=False):
        x = _f32(x); q = np.ascontiguousarray(q, np.int8); scale = _f32(scale)
        S, I = x.shape; O = q.shape[0]
        y = np.empty((S, O), np.float32)
        acc = np.empty((S, O), np.int32) if want_acc else None
        self.lib.oracle_matmul_q_s(_p(y), _p(x), _p(q), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O),
                                   _p(acc), None, None)
        return (y, acc) if want_acc else y

    def matmul_i4_idot_s(self, x, q4, scale, I):
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); scale = _f32(scale)
        S = x.shape[0]; O = scale.size
        y = np.empty((S, O), np.float32)
        self.lib.oracle_matmul_i4_idot_s(_p(y), _p(x), _p(q4), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def attn_core(self, q, k, v, pos_base, cache):
        """nn/attn.c:29-74 without projections: QK-norm + RoPE (q, k are modified in place), KV store into
        ``cache`` (an AttnCache), scores / softmax / accumulation.  q [S][H*hd], k, v [S][KV*hd] -> ctx [S][H*hd]."""
        c = cache
        q = _f32(q); k = _f32(k); v = _f32(v); S = q.shape[0]
        ctx = np.empty_like(q)
        null = C.c_void_p(0)
        if c.gemma:
            one = np.float32(1)
            mul = lambda w: None if w is None else (one + w).astype(np.float32)      # the (1 + w) multipliers, in f32
            qn, kn, vn = mul(c.qn), mul(c.kn), mul(c.vn)
            self.lib.oracle_attn_core_gemma(_p(ctx), _p(q), _p(k), _p(v), C.c_int(S), C.c_int(pos_base), C.c_int(c.H), C.c_int(c.KV),
                                            C.c_int(c.hd), C.c_float(c.theta), C.c_float(c.eps), C.c_int(c.rot),
                                            _p(qn) if qn is not None else null, _p(kn) if kn is not None else null,
                                            _p(vn) if vn is not None else null, C.c_int(c.window), C.c_float(c.scale),
                                            _p(c.K) if not c.kv8 else null, _p(c.V) if not c.kv8 else null,
                                            _p(c.K8) if c.kv8 else null, _p(c.V8) if c.kv8 else null,
                                            _p(c.Ks) if c.kv8 else null, _p(c.Vs) if c.kv8 else null, C.c_int(c.max_t))
            return ctx
        self.lib.oracle_attn_core(_p(ctx), _p(q), _p(k), _p(v), C.c_int(S), C.c_int(pos_base), C.c_int(c.H), C.c_int(c.KV),
                                  C.c_int(c.hd), C.c_float(c.theta), C.c_float(c.eps), C.c_int(c.rot),
                                  _p(c.qn) if c.qn is not None else null, _p(c.kn) if c.kn is not None else null,
                                  _p(c.K) if not c.kv8 else null, _p(c.V) if not c.kv8 else null,
                                  _p(c.K8) if c.kv8 else null, _p(c.V8) if c.kv8 else null,
                                  _p(c.Ks) if c.kv8 else null, _p(c.Vs) if c.kv8 else null, C.c_int(c.max_t))
        return ctx

    def pack_int4_grouped(self, w, gs=32):
        w = _f32(w); O, I = w.shape
        q4 = np.empty((O, (I + 1) // 2), np.uint8); s = np.empty((O, (I + gs - 1) // gs), np.float32)
        self.lib.oracle_pack_int4_grouped(_p(w), _p(q4), _p(s), C.c_int(O), C.c_int(I), C.c_int(gs))
        return q4, s

    def matmul_i4g_idot_s(self, x, q4, scale):
        """WF_I4G, group 32, integer path (IDOT4=1): x [S][I], q4 [O][I/2], scale [O][I/32]."""
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); scale = _f32(scale)
        S, I = x.shape; O = scale.shape[0]
        y = np.empty((S, O), np.float32)
        self.lib.oracle_matmul_i4g_idot_s(_p(y), _p(x), _p(q4), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def matmul_i4g_f32_s(self, x, q4, scale):
        """WF_I4G, group 32, the reference's default product (no IDOT4): f32 x dequantized int4."""
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); scale = _f32(scale)
        S, I = x.shape; O = scale.shape[0]
        y = np.empty((S, O), np.float32)
        self.lib.oracle_matmul_i4g_f32_s(_p(y), _p(x), _p(q4), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def matmul_q4r4_s(self, x, q4, s16, O):
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); s16 = np.ascontiguousarray(s16, np.uint16)
        S, I = x.shape
        y = np.empty((S, O), np.float32)
        self.lib.oracle_matmul_q4r4_s(_p(y), _p(x), _p(q4), _p(s16), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def q4r4_gemm(self, w, d, xq, xs, xsum, nb, ns):
        """One 4-row block; returns (y [ns][4], int32 group sums [ns][4][nb])."""
        y = np.empty((ns, 4), np.float32)
        isum = np.empty((ns, 4, nb), np.int32)
        self.lib.oracle_q4r4_gemm(_p(np.ascontiguousarray(w)), _p(np.ascontiguousarray(d)), _p(np.ascontiguousarray(xq)),
                                  _p(np.ascontiguousarray(xs)), _p(np.ascontiguousarray(xsum)),
                                  C.c_int(nb), C.c_int(ns), _p(y), C.c_int(4), _p(isum))
        return y, isum

    # -- load-time quantizers ------------------------------------------
    def quantize_rows(self, w, bits=8):
        w = _f32(w); O, I = w.shape
        q = np.empty((O, I), np.int8); s = np.empty(O, np.float32)
        self.lib.oracle_quantize_rows(_p(w), _p(q), _p(s), C.c_int(O), C.c_int(I), C.c_int(bits))
        return q, s

    def pack_int4(self, w):
        w = _f32(w); O, I = w.shape
        q4 = np.empty((O, (I + 1) // 2), np.uint8); s = np.empty(O, np.float32)
        self.lib.oracle_pack_int4(_p(w), _p(q4), _p(s), C.c_int(O), C.c_int(I))
        return q4, s

    def pack_q4r4(self, w):
        w = _f32(w); O, I = w.shape
        nblk, nb = (O + 3) // 4, I // 32
        q4 = np.empty(nblk * nb * 64, np.uint8); s16 = np.empty(nblk * nb * 4, np.uint16)
        self.lib.oracle_pack_q4r4(_p(w), C.c_int(O), C.c_int(I), _p(q4), _p(s16))
        return q4, s16

    def pack_q8r4(self, w):
        w = _f32(w); O, I = w.shape
        nblk, nb = (O + 3) // 4, I // 32
        q8 = np.empty(nblk * nb * 128, np.int8); s16 = np.empty(nblk * nb * 4, np.uint16)
        self.lib.oracle_pack_q8r4(_p(w), C.c_int(O), C.c_int(I), _p(q8), _p(s16))
        return q8, s16

    def matmul_q8r4_s(self, x, q8, s16, O):
        x = _f32(x); q8 = np.ascontiguousarray(q8, np.int8); s16 = np.ascontiguousarray(s16, np.uint16)
        S, I = x.shape
        y = np.empty((S, O), np.float32)
        self.lib.oracle_matmul_q8r4_s(_p(y), _p(x), _p(q8), _p(s16), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    # -- router ---------------------------------------------------------
    def softmax(self, x):
        x = _f32(x).copy()
        rows = x.reshape(-1, x.shape[-1])
        for r in range(rows.shape[0]):
            self.lib.oracle_softmax(_p(rows[r]), C.c_int(rows.shape[1]))
        return x

    def moe_topk(self, p, K, norm):
        p = _f32(p); rows = p.reshape(-1, p.shape[-1])
        idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
        for r in range(rows.shape[0]):
            self.lib.oracle_moe_topk(_p(rows[r]), C.c_int(rows.shape[1]), C.c_int(K), _p(idx[r]), _p(w[r]), C.c_int(norm))
        return idx, w

    def route_topk(self, logits, K):
        lg = _f32(logits).copy(); rows = lg.reshape(-1, lg.shape[-1])
        idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
        for r in range(rows.shape[0]):
            self.lib.oracle_route_topk(_p(rows[r]), C.c_int(rows.shape[1]), C.c_int(K), _p(idx[r]), _p(w[r]))
        return idx, w, lg

    def argmax(self, v):
        v = _f32(v)
        return int(self.lib.oracle_argmax(_p(v), C.c_int(v.size)))

    # -- blocks ---------------------------------------------------------
    def silu_mul(self, g, u):
        g = _f32(g).copy(); u = _f32(u)
        self.lib.oracle_silu_mul(_p(g), _p(u), C.c_int64(g.size))
        return g

    def gelu_mul(self, g, u):
        g = _f32(g).copy(); u = _f32(u)
        self.lib.oracle_gelu_mul(_p(g), _p(u), C.c_int64(g.size))
        return g

    def ffn_q8(self, x, gq, gs, uq, us, dq, ds, act=0, want_h=False):
        x = _f32(x); S, D = x.shape; I = gq.shape[0]
        out = np.empty((S, D), np.float32)
        h = np.empty((S, I), np.float32) if want_h else None
        self.lib.oracle_ffn_q8(_p(out), _p(x), C.c_int(S), C.c_int(D), C.c_int(I), C.c_int(act),
                               _p(gq), _p(_f32(gs)), _p(uq), _p(_f32(us)), _p(dq), _p(_f32(ds)), _p(h))
        return (out, h) if want_h else out

    def ffn_q4r4(self, x, I, gq, gs, uq, us, dq, ds, act=0):
        x = _f32(x); S, D = x.shape
        out = np.empty((S, D), np.float32)
        self.lib.oracle_ffn_q4r4(_p(out), _p(x), C.c_int(S), C.c_int(D), C.c_int(I), C.c_int(act),
                                 _p(gq), _p(gs), _p(uq), _p(us), _p(dq), _p(ds))
        return out

    def _moe(self, fn, ex, x, logits, *extra):
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        fn(C.byref(ex.c), _p(x), *extra[:1], _p(lg), _p(out), *extra[1:], _p(idx), _p(w))
        return out, idx, w

    def moe_d1(self, ex, x, logits):
        x = _f32(x).reshape(1, ex.D); lg = _f32(logits).reshape(1, ex.E).copy()
        out = np.empty((1, ex.D), np.float32)
        idx = np.empty((1, ex.K), np.int32); w = np.empty((1, ex.K), np.float32)
        self.lib.oracle_moe_d1(C.byref(ex.c), _p(x), _p(lg), _p(out), _p(idx), _p(w))
        return out, idx, w

    def moe_batch(self, ex, x, logits):
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        self.lib.oracle_moe_batch(C.byref(ex.c), _p(x), C.c_int(S), _p(lg), _p(out), _p(idx), _p(w))
        return out, idx, w

    def moe_sigmoid(self, ex, x, logits, bias=None):
        """The block behind the sigmoid + expert-bias gate (nn/moe.c:10-25): S = 1 decode order, S > 1 batch order."""
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        b = None if bias is None else _f32(bias)
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        if S == 1:
            self.lib.oracle_moe_sigmoid_d1(C.byref(ex.c), _p(x), _p(lg), _p(b), _p(out), _p(idx), _p(w))
        else:
            self.lib.oracle_moe_sigmoid_batch(C.byref(ex.c), _p(x), C.c_int(S), _p(lg), _p(b), _p(out), _p(idx), _p(w))
        return out, idx, w

    def olmoe_moe(self, ex, x, logits, norm_topk):
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        self.lib.oracle_olmoe_moe(C.byref(ex.c), _p(x), C.c_int(S), _p(lg), _p(out), C.c_int(norm_topk), _p(idx), _p(w))
        return out, idx, w

    def moe_q4r4(self, ex, x, logits):
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        self.lib.oracle_moe_q4r4(C.byref(ex.c), _p(x), C.c_int(S), _p(lg), _p(out), _p(idx), _p(w))
        return out, idx, w


class Ref:
    """The unmodified reference, compiled by oracle/Makefile.  ``Ref.available()``
    is False where neither the sources nor a prebuilt library exist."""

    @staticmethod
    def path():
        d = os.path.join(HERE, "_ref")
        native = os.path.join(d, "libmoty_ref_native.so")
        v3 = os.path.join(d, "libmoty_ref_v3.so")
        need = os.path.join(d, "native_needs_avx512vnni")
        if os.path.exists(native):
            needs512 = os.path.exists(need) and open(need).read().strip() not in ("", "0")
            if not needs512 or (_cpu_has("avx512_vnni") and _cpu_has("avx512bw")):
                return native
        return v3 if os.path.exists(v3) else None

    @staticmethod
    def available():
        return Ref.path() is not None

    def __init__(self, threads: int | None = None):
        p = Ref.path()
        if p is None:
            raise RuntimeError("reference library not built (oracle/_ref is empty)")
        self.tier = "native" if p.endswith("native.so") else "x86-64-v3"
        os.environ.setdefault("MOTY_NO_OMP_TUNE", "1")
        os.environ.setdefault("IDOT4", "1")      # the int4 drivers read it once, on their first call
        self.lib = C.CDLL(p)
        L = self.lib
        L.moty_hw_qrow_i8.restype = C.c_float
        L.moty_hw_dot_i8i8.restype = C.c_int32
        L.moty_hw_dot_i4i8.restype = C.c_int32
        L.moty_hw_f16_to_f32.restype = C.c_float
        L.moty_hw_f16_to_f32.argtypes = [C.c_uint16]
        L.moty_f32_to_f16.restype = C.c_uint16
        L.moty_f32_to_f16.argtypes = [C.c_float]
        L.moty_argmax_v.restype = C.c_int
        L.refshim_threads.restype = C.c_int
        if threads:
            L.refshim_set_threads(C.c_int(threads))

    def threads(self):
        return int(self.lib.refshim_threads())

    def set_threads(self, n):
        self.lib.refshim_set_threads(C.c_int(n))

    def f16_to_f32(self, h):
        return self.lib.moty_hw_f16_to_f32(int(h))

    def f32_to_f16(self, f):
        return self.lib.moty_f32_to_f16(float(np.float32(f)))

    def qrow_i8(self, x):
        x = _f32(x); q = np.empty(x.shape, np.int8)
        s = self.lib.moty_hw_qrow_i8(_p(x), _p(q), C.c_int(x.size))
        return q, np.float32(s)

    def quant_g32(self, x):
        x = _f32(x); I = x.shape[-1]; rows = x.reshape(-1, I)
        xq = np.empty(rows.shape, np.int8)
        xs = np.empty((rows.shape[0], I // 32), np.float32); xsum = np.empty((rows.shape[0], I // 32), np.int32)
        for r in range(rows.shape[0]):
            self.lib.moty_hw_quant_g32(_p(rows[r]), C.c_int(I), _p(xq[r]), _p(xs[r]), _p(xsum[r]))
        return xq, xs, xsum

    def dot_i8i8(self, w, x):
        w = np.ascontiguousarray(w, np.int8); x = np.ascontiguousarray(x, np.int8)
        return int(self.lib.moty_hw_dot_i8i8(_p(w), _p(x), C.c_int(w.size)))

    def dot_i4i8(self, w4, x):
        w4 = np.ascontiguousarray(w4, np.uint8); x = np.ascontiguousarray(x, np.int8)
        return int(self.lib.moty_hw_dot_i4i8(_p(w4), _p(x), C.c_int(x.size)))

    def matmul_q_s(self, x, q, scale):
        x = _f32(x); q = np.ascontiguousarray(q, np.int8); scale = _f32(scale)
        S, I = x.shape; O = q.shape[0]
        y = np.empty((S, O), np.float32)
        self.lib.moty_matmul_q_s(_p(y), _p(x), _p(q), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def matmul_q4r4_s(self, x, q4, s16, O):
        x = _f32(x); S, I = x.shape
        y = np.empty((S, O), np.float32)
        self.lib.moty_matmul_q4r4_s(_p(y), _p(x), _p(np.ascontiguousarray(q4, np.uint8)),
                                    _p(np.ascontiguousarray(s16, np.uint16)), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def quantize_rows(self, w, bits=8):
        w = _f32(w); O, I = w.shape
        q = np.empty((O, I), np.int8); s = np.empty(O, np.float32)
        self.lib.moty_quantize_rows(_p(w), _p(q), _p(s), C.c_int(O), C.c_int(I), C.c_int(bits))
        return q, s

    def pack_int4(self, w):
        w = _f32(w); O, I = w.shape
        q4 = np.empty((O, (I + 1) // 2), np.uint8); s = np.empty(O, np.float32)
        self.lib.moty_pack_int4(_p(w), _p(q4), _p(s), C.c_int(O), C.c_int(I))
        return q4, s

    def attn_core(self, q, k, v, pos_base, cache):
        """The same steps through the reference's own functions, composed as attn_tail does (nn/attn.c:29-74):
        moty_rmsnorm_row, moty_rope_head, memcpy / moty_kv_store_row, moty_att_scores_*, moty_softmax_row,
        moty_att_accum_*."""
        c = cache; L = self.lib
        q = _f32(q); k = _f32(k); v = _f32(v); S = q.shape[0]; hd = c.hd; G = c.H // c.KV
        if c.gemma:
            # engines/gemma.c:299-386 through the engine's own static gnorm_row / gemma_rope_head (zc_norm gains 1 + w)
            def gn(row, w):
                L.refshim_gemma_gnorm_row(C.c_int(1), C.c_float(c.eps), _p(row), _p(row), _p(w), C.c_int(hd))
            def rope(row, pos):
                L.refshim_gemma_rope_head(_p(row), C.c_int(pos), C.c_float(c.theta), C.c_int(hd), C.c_int(c.rot))
            for s in range(S):
                for hh in range(c.KV):
                    row = k[s, hh * hd:(hh + 1) * hd]
                    if c.kn is not None:
                        gn(row, c.kn)
                    if c.vn is not None:
                        gn(v[s, hh * hd:(hh + 1) * hd], c.vn)
                    rope(row, pos_base + s)
                for hh in range(c.H):
                    row = q[s, hh * hd:(hh + 1) * hd]
                    if c.qn is not None:
                        gn(row, c.qn)
                    rope(row, pos_base + s)
        for s in range(S if not c.gemma else 0):
            for hh in range(c.H):
                row = q[s, hh * hd:(hh + 1) * hd]
                if c.qn is not None:
                    L.moty_rmsnorm_row(_p(row), _p(row), _p(c.qn), C.c_int(hd), C.c_float(c.eps))
                L.moty_rope_head(_p(row), C.c_int(pos_base + s), C.c_float(c.theta), C.c_int(c.rot))
            for hh in range(c.KV):
                row = k[s, hh * hd:(hh + 1) * hd]
                if c.kn is not None:
                    L.moty_rmsnorm_row(_p(row), _p(row), _p(c.kn), C.c_int(hd), C.c_float(c.eps))
                L.moty_rope_head(_p(row), C.c_int(pos_base + s), C.c_float(c.theta), C.c_int(c.rot))
        for s in range(S):
            for hh in range(c.KV):
                t = pos_base + s
                if c.kv8:
                    sc = C.c_float(0)
                    L.moty_kv_store_row(_p(c.K8[hh, t]), C.byref(sc), _p(k[s, hh * hd:(hh + 1) * hd]), C.c_int(hd)); c.Ks[hh, t] = sc.value
                    L.moty_kv_store_row(_p(c.V8[hh, t]), C.byref(sc), _p(v[s, hh * hd:(hh + 1) * hd]), C.c_int(hd)); c.Vs[hh, t] = sc.value
                else:
                    c.K[hh, t] = k[s, hh * hd:(hh + 1) * hd]; c.V[hh, t] = v[s, hh * hd:(hh + 1) * hd]
        ctx = np.empty_like(q)
        scale = C.c_float(np.float32(c.scale) if c.scale > 0 else np.float32(1.0) / np.sqrt(np.float32(hd)))
        for hh in range(c.H):
            for s in range(S):
                qpos = pos_base + s; kvh = hh // G
                t0 = max(0, qpos - c.window + 1) if c.window > 0 else 0          # engines/gemma.c:373
                sc = np.empty(qpos - t0 + 1, np.float32); cx = np.empty(hd, np.float32)
                qv = np.ascontiguousarray(q[s, hh * hd:(hh + 1) * hd])
                base = C.c_int64(kvh * c.max_t)
                if c.kv8:
                    L.moty_att_scores_i8(_p(sc), _p(qv), _p(c.K8), _p(c.Ks), base, C.c_int(t0), C.c_int(qpos), C.c_int(hd), scale)
                else:
                    L.moty_att_scores_f32(_p(sc), _p(qv), _p(c.K), base, C.c_int(t0), C.c_int(qpos), C.c_int(hd), scale)
                L.moty_softmax_row(_p(sc), C.c_int(qpos - t0 + 1))
                if c.kv8:
                    L.moty_att_accum_i8(_p(cx), _p(sc), _p(c.V8), _p(c.Vs), base, C.c_int(t0), C.c_int(qpos), C.c_int(hd))
                else:
                    L.moty_att_accum_f32(_p(cx), _p(sc), _p(c.V), base, C.c_int(t0), C.c_int(qpos), C.c_int(hd))
                ctx[s, hh * hd:(hh + 1) * hd] = cx
        return ctx

    def pack_int4_grouped(self, w, gs=32):
        w = _f32(w); O, I = w.shape
        q4 = np.empty((O, (I + 1) // 2), np.uint8); s = np.empty((O, (I + gs - 1) // gs), np.float32)
        self.lib.moty_pack_int4_grouped(_p(w), _p(q4), _p(s), C.c_int(O), C.c_int(I), C.c_int(gs))
        return q4, s

    def has_i4g_idot(self):
        """The reference takes the integer path of WF_I4G only in builds with AVX512-VNNI (nn/matmul.c:168)."""
        return self.tier == "native" and _cpu_has("avx512_vnni")

    def matmul_i4g_idot_s(self, x, q4, scale):
        """moty_matmul_i4_grouped_s with IDOT4=1 (set before the library is loaded), gs = 32, I % 64 == 0."""
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); scale = _f32(scale)
        S, I = x.shape; O = scale.shape[0]
        assert I % 64 == 0 and self.has_i4g_idot()
        y = np.empty((S, O), np.float32)
        self.lib.moty_matmul_i4_grouped_s(_p(y), _p(x), _p(q4), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(32))
        return y

    def matmul_i4g_any(self, x, q4, scale):
        """moty_matmul_i4_grouped_s as the process's IDOT4 setting and the shape select it (gs = 32): rows that are not a
        multiple of 64 always take the f32 x int4 product (nn/matmul.c:172), whatever IDOT4 says."""
        x = _f32(x); q4 = np.ascontiguousarray(q4, np.uint8); scale = _f32(scale)
        S, I = x.shape; O = scale.shape[0]
        y = np.empty((S, O), np.float32)
        self.lib.moty_matmul_i4_grouped_s(_p(y), _p(x), _p(q4), _p(scale), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(32))
        return y


    def pack_q4r4(self, w):
        w = _f32(w); O, I = w.shape
        nblk, nb = (O + 3) // 4, I // 32
        q4 = np.empty(nblk * nb * 64, np.uint8); s16 = np.empty(nblk * nb * 4, np.uint16)
        self.lib.refshim_pack_q4r4(_p(w), C.c_int(O), C.c_int(I), _p(q4), _p(s16))
        return q4, s16

    def pack_q8r4(self, w):
        w = _f32(w); O, I = w.shape
        nblk, nb = (O + 3) // 4, I // 32
        q8 = np.empty(nblk * nb * 128, np.int8); s16 = np.empty(nblk * nb * 4, np.uint16)
        self.lib.refshim_pack_q8r4(_p(w), C.c_int(O), C.c_int(I), _p(q8), _p(s16))
        return q8, s16

    def matmul_q8r4_s(self, x, q8, s16, O):
        x = _f32(x); S, I = x.shape
        y = np.empty((S, O), np.float32)
        self.lib.moty_matmul_q8r4_s(_p(y), _p(x), _p(np.ascontiguousarray(q8, np.int8)),
                                    _p(np.ascontiguousarray(s16, np.uint16)), C.c_int(S), C.c_int(I), C.c_int(O))
        return y

    def softmax(self, x):
        x = _f32(x).copy(); rows = x.reshape(-1, x.shape[-1])
        for r in range(rows.shape[0]):
            self.lib.moty_softmax_row(_p(rows[r]), C.c_int(rows.shape[1]))
        return x

    def moe_topk(self, p, K, norm):
        p = _f32(p); rows = p.reshape(-1, p.shape[-1])
        idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
        for r in range(rows.shape[0]):
            self.lib.moty_moe_topk(_p(rows[r]), C.c_int(rows.shape[1]), C.c_int(K), _p(idx[r]), _p(w[r]), C.c_int(norm))
        return idx, w

    def route_topk(self, logits, K):
        lg = _f32(logits).copy(); rows = lg.reshape(-1, lg.shape[-1])
        idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
        for r in range(rows.shape[0]):
            self.lib.refshim_route_topk(_p(rows[r]), C.c_int(rows.shape[1]), C.c_int(K), _p(idx[r]), _p(w[r]))
        return idx, w, lg

    def argmax(self, v):
        v = _f32(v)
        return int(self.lib.moty_argmax_v(_p(v), C.c_int(v.size)))

    def silu_mul(self, g, u):
        g = _f32(g).copy(); u = _f32(u)
        self.lib.moty_hw_silu_mul(_p(g), _p(u), C.c_int64(g.size))
        return g

    def moe_topk_block(self, ex, x, router_f=None, router_q=None, router_qs=None):
        """nn/moe.c block (S=1: decode path, S>1: batch path); router f32 or int8."""
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        out = np.empty((S, ex.D), np.float32)
        fmt = WF_F32 if router_f is not None else WF_I8
        self.lib.refshim_moe_topk(C.byref(ex.c), C.c_int(fmt), _p(_f32(router_f)) if router_f is not None else None,
                                  _p(router_q) if router_q is not None else None,
                                  _p(_f32(router_qs)) if router_qs is not None else None,
                                  _p(x), C.c_int(S), _p(out))
        return out

    def gelu_mul(self, g, u):
        """g = gelu_tanh(g) * u with the engine's own static gelu_tanh (engines/gemma.c:389-391,398)."""
        g = _f32(g).copy(); u = _f32(u)
        self.lib.refshim_gemma_gelu_mul(_p(g), _p(u), C.c_int64(g.size))
        return g

    def gemma_gnorm_row(self, x, w, eps=1e-6, zc_norm=True):
        x = _f32(x); out = np.empty_like(x)
        self.lib.refshim_gemma_gnorm_row(C.c_int(int(zc_norm)), C.c_float(eps), _p(out), _p(x), _p(_f32(w)), C.c_int(x.size))
        return out

    def gemma_rope_head(self, x, pos, theta, rot_angles):
        x = _f32(x).copy()
        self.lib.refshim_gemma_rope_head(_p(x), C.c_int(pos), C.c_float(theta), C.c_int(x.size), C.c_int(rot_angles))
        return x

    def moe_sigmoid_block(self, ex, x, bias, router_q, router_qs):
        """nn/moe.c block behind the sigmoid + bias gate, int8 router."""
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        out = np.empty((S, ex.D), np.float32)
        self.lib.refshim_moe_sigmoid(C.byref(ex.c), C.c_int(WF_I8), None, _p(router_q), _p(_f32(router_qs)),
                                     _p(_f32(bias)) if bias is not None else None, _p(x), C.c_int(S), _p(out))
        return out

    def moe_i4_block(self, ex4, x, router_q, router_qs, sig=False, bias=None):
        """nn/moe.c block over per-row int4 experts (ebits = 4; ``ex4`` is an Experts whose g / u / d hold the nibble
        rows [E][I][(D+1)/2], [E][I][(D+1)/2], [E][D][(I+1)/2]), softmax or sigmoid gate, int8 router.  The batch path
        (S > 1) is integer only with IDOT4=1, which this module sets before the library is loaded."""
        x = _f32(x).reshape(-1, ex4.D); S = x.shape[0]
        out = np.empty((S, ex4.D), np.float32)
        self.lib.refshim_moe_i4(C.byref(ex4.c), C.c_int(WF_I8), None, _p(router_q), _p(_f32(router_qs)), C.c_int(1 if sig else 0),
                                _p(_f32(bias)) if bias is not None else None, _p(x), C.c_int(S), _p(out))
        return out

    def olmoe_moe(self, ex, x, logits, norm_topk):
        x = _f32(x).reshape(-1, ex.D); S = x.shape[0]
        lg = _f32(logits).reshape(S, ex.E).copy()
        out = np.empty((S, ex.D), np.float32)
        idx = np.empty((S, ex.K), np.int32); w = np.empty((S, ex.K), np.float32)
        self.lib.refshim_olmoe_moe(C.byref(ex.c), _p(x), C.c_int(S), _p(lg), _p(out), C.c_int(norm_topk), _p(idx), _p(w))
        return out, idx, w

    def dense_ffn(self, fmt, x, I, gq, gs, uq, us, dq, ds):
        x = _f32(x); S, D = x.shape
        out = np.empty((S, D), np.float32)
        self.lib.refshim_dense_ffn(C.c_int(fmt), _p(gq), _p(gs), _p(uq), _p(us), _p(dq), _p(ds),
                                   C.c_int(D), C.c_int(I), _p(x), C.c_int(S), _p(out))
        return out
