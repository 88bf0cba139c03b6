"""moty_b200 -- host-side mirror of moty's quantized-matmul operators over the
sm_100a library ``libmoty_cuda.so`` (C ABI in ``include/moty_cuda.h``).

Names follow the reference's operator layer (moty source tree, directory c/):
``Mat`` + ``mat_apply`` (nn/nn_mat.h:18-30, nn/mat.c:70-83), ``dense_ffn``
(nn/ffn.h:14), the MoE block (nn/moe.h:35-38), the hw.h kernels (hw/hw.h:58-124).
Arrays are numpy; shapes follow the reference: x ``[S][I]``, y ``[S][O]``.

There is no CPU fallback: if the library is missing or a call fails, an
exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmoty_cuda.so")

WF_F32, WF_I8, WF_I4, WF_I4G, WF_Q4R4, WF_Q8R4 = 0, 1, 2, 4, 7, 8
ACT_SILU, ACT_GELU_TANH = 0, 1
QROW_MAX = 16384

_lib = None


class MotyCudaError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MotyCudaError(f"{LIB_PATH} is missing: build it with `python -m moty_b200.build` "
                                "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH)
        _lib.moty_cuda_last_error.restype = C.c_char_p
        _lib.moty_cuda_mat_bytes.restype = C.c_int64
    return _lib


def _ck(rc: int) -> None:
    if rc != 0:
        raise MotyCudaError(f"libmoty_cuda error {rc}: {lib().moty_cuda_last_error().decode()}")


def _p(a):
    if a is None:
        return None
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("array must be C-contiguous")
    return C.c_void_p(a.ctypes.data)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def init(devices=None) -> None:
    """moty_cuda_init: select GPUs (default: device 0)."""
    if devices is None:
        _ck(lib().moty_cuda_init(None, 0))
    else:
        arr = (C.c_int * len(devices))(*devices)
        _ck(lib().moty_cuda_init(arr, len(devices)))


CUDA_STREAM_LEGACY = 1        # cudaStreamLegacy: the handle that NAMES the default stream (0 means "the library's own")


def stream_handle(torch_stream) -> int:
    """The handle to pass as `stream` for a torch stream.  torch reports the default stream as 0, which the
    library reads as "my own stream" -- work there would not be ordered with the caller's default-stream work --
    so the default stream is passed by its explicit name instead."""
    h = int(torch_stream.cuda_stream)
    return h if h != 0 else CUDA_STREAM_LEGACY


def shutdown() -> None:
    lib().moty_cuda_shutdown()


def sync(device: int = 0) -> None:
    _ck(lib().moty_cuda_sync(device))


def sm_count(device: int = 0) -> int:
    n = lib().moty_cuda_sm_count(device)
    if n < 0:
        _ck(n)
    return n


def pinned_empty(shape, dtype) -> np.ndarray:
    """A numpy array in page-locked host memory (freed when the array dies)."""
    dtype = np.dtype(dtype)
    n = int(np.prod(shape)) * dtype.itemsize
    ptr = C.c_void_p()
    _ck(lib().moty_cuda_host_alloc(C.byref(ptr), C.c_size_t(max(n, 1))))
    buf = (C.c_char * max(n, 1)).from_address(ptr.value)
    arr = np.frombuffer(buf, dtype=dtype, count=int(np.prod(shape))).reshape(shape)
    _PINNED[arr.ctypes.data] = ptr.value
    return arr


_PINNED: dict[int, int] = {}


def pinned_free(arr: np.ndarray) -> None:
    p = _PINNED.pop(arr.ctypes.data, None)
    if p:
        _ck(lib().moty_cuda_host_free(C.c_void_p(p)))


# ---------------------------------------------------------------------------
# weights and mat_apply
# ---------------------------------------------------------------------------
class Mat:
    """A weight matrix resident on one GPU (the device-side ``Mat``)."""

    def __init__(self, fmt: int, codes: np.ndarray, scales, O: int, I: int, device: int = 0, rows=None):
        self.fmt, self.O, self.I, self.device = fmt, O, I, device
        codes = np.ascontiguousarray(codes)
        scales = None if scales is None else np.ascontiguousarray(scales)
        h = C.c_void_p()
        if rows is None:
            _ck(lib().moty_cuda_upload_mat(C.byref(h), fmt, _p(codes), _p(scales), O, I, device))
        else:
            _ck(lib().moty_cuda_upload_mat_rows(C.byref(h), fmt, _p(codes), _p(scales), O, I, rows[0], rows[1], device))
            self.O = rows[1] - rows[0]
        self.h = h

    @classmethod
    def i8(cls, q, scale, device=0, rows=None):
        q = np.ascontiguousarray(q, np.int8)
        return cls(WF_I8, q, _f32(scale), q.shape[0], q.shape[1], device, rows)

    @classmethod
    def q4r4(cls, q4, s16, O, I, device=0, rows=None):
        return cls(WF_Q4R4, np.ascontiguousarray(q4, np.uint8), np.ascontiguousarray(s16, np.uint16), O, I, device, rows)

    @classmethod
    def q8r4(cls, q8, s16, O, I, device=0, rows=None):
        return cls(WF_Q8R4, np.ascontiguousarray(q8, np.int8), np.ascontiguousarray(s16, np.uint16), O, I, device, rows)

    @classmethod
    def i4(cls, q4, scale, O, I, device=0, rows=None):
        """WF_I4: q4 [O][(I+1)/2] (even element in the low nibble), scale f32 [O]."""
        return cls(WF_I4, np.ascontiguousarray(q4, np.uint8), _f32(scale), O, I, device, rows)

    @classmethod
    def i4g(cls, q4, scale, O, I, device=0):
        """WF_I4G: q4 [O][I/2] (even element in the low nibble), scale f32 [O][I/32]; group size 32."""
        return cls(WF_I4G, np.ascontiguousarray(q4, np.uint8), _f32(scale), O, I, device)

    @classmethod
    def f32(cls, w, device=0):
        w = _f32(w)
        return cls(WF_F32, w, None, w.shape[0], w.shape[1], device)

    def nbytes(self) -> int:
        return int(lib().moty_cuda_mat_bytes(self.h))

    def free(self) -> None:
        if self.h:
            lib().moty_cuda_free_mat(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def mat_apply(w: Mat, x, y: np.ndarray | None = None, want_acc: bool = False):
    """moty_mat_apply (nn/mat.c:70-83) with host arrays: returns y ``[S][O]``
    (and the int32 accumulators for WF_I8 when ``want_acc``)."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    S = x.shape[0]
    if x.shape[1] != w.I:
        raise ValueError(f"x has width {x.shape[1]}, matrix expects {w.I}")
    if y is None:
        y = np.empty((S, w.O), np.float32)
    if want_acc:
        acc = np.empty((S, w.O), np.int32)
        _ck(lib().moty_cuda_mat_apply_acc(w.h, _p(y), _p(acc), _p(x), S))
        return y, acc
    _ck(lib().moty_cuda_mat_apply(w.h, _p(y), _p(x), S))
    return y


def mat_apply_dev(w: Mat, y_ptr: int, x_ptr: int, S: int, stream: int = 0) -> None:
    """Device-pointer form: enqueue only (no synchronisation)."""
    _ck(lib().moty_cuda_mat_apply_dev(w.h, C.c_void_p(y_ptr), C.c_void_p(x_ptr), S, C.c_void_p(stream)))


def mat_apply_multi_dev(ws, y_ptrs, x_ptrs, stream: int = 0) -> None:
    """Up to eight independent one-row Q8_0 products in one launch (device pointers)."""
    n = len(ws)
    _ck(lib().moty_cuda_mat_apply_multi_dev(n, (C.c_void_p * n)(*[w.h.value for w in ws]),
                                            (C.c_void_p * n)(*y_ptrs), (C.c_void_p * n)(*x_ptrs), C.c_void_p(stream)))


def matmul_q_s(x, q, scale):
    """moty_matmul_q_s (nn/matmul.c:51-66) with host weights."""
    x = _f32(x); q = np.ascontiguousarray(q, np.int8); scale = _f32(scale)
    S, I = x.shape; O = q.shape[0]
    y = np.empty((S, O), np.float32)
    _ck(lib().moty_cuda_matmul_q_s(_p(y), _p(x), _p(q), _p(scale), S, I, O))
    return y


def matmul_q4r4_s(x, q4, s16, O):
    """moty_matmul_q4r4_s (nn/matmul.c:405-433) with host weights."""
    x = _f32(x); S, I = x.shape
    y = np.empty((S, O), np.float32)
    _ck(lib().moty_cuda_matmul_q4r4_s(_p(y), _p(x), _p(np.ascontiguousarray(q4, np.uint8)),
                                      _p(np.ascontiguousarray(s16, np.uint16)), S, I, O))
    return y


def matmul_i4_grouped_s(x, q4, scale, O, gs=32):
    """moty_matmul_i4_grouped_s (nn/matmul.c:164-197, integer path) with host weights."""
    x = _f32(x); S, I = x.shape
    y = np.empty((S, O), np.float32)
    _ck(lib().moty_cuda_matmul_i4_grouped_s(_p(y), _p(x), _p(np.ascontiguousarray(q4, np.uint8)), _p(_f32(scale)),
                                            S, I, O, gs))
    return y


def matmul_q8r4_s(x, q8, s16, O):
    """moty_matmul_q8r4_s (nn/matmul.c:435-461) with host weights."""
    x = _f32(x); S, I = x.shape
    y = np.empty((S, O), np.float32)
    _ck(lib().moty_cuda_matmul_q8r4_s(_p(y), _p(x), _p(np.ascontiguousarray(q8, np.int8)),
                                      _p(np.ascontiguousarray(s16, np.uint16)), S, I, O))
    return y


# ---------------------------------------------------------------------------
# hw.h kernels
# ---------------------------------------------------------------------------
def qrow_i8(x):
    """moty_hw_qrow_i8 per row: returns (q int8 [rows][n], scale f32 [rows])."""
    x = _f32(x)
    rows = x.reshape(-1, x.shape[-1]) if x.ndim > 1 else x[None, :]
    q = np.empty(rows.shape, np.int8); s = np.empty(rows.shape[0], np.float32)
    _ck(lib().moty_cuda_qrow_i8(_p(rows), _p(q), _p(s), rows.shape[0], rows.shape[1]))
    return q.reshape(x.shape), s


def quant_g32(x):
    """moty_hw_quant_g32 per row: (xq, xs [rows][I/32], xsum [rows][I/32])."""
    x = _f32(x)
    rows = x.reshape(-1, x.shape[-1])
    I = rows.shape[1]
    xq = np.empty(rows.shape, np.int8)
    xs = np.empty((rows.shape[0], I // 32), np.float32); xsum = np.empty((rows.shape[0], I // 32), np.int32)
    _ck(lib().moty_cuda_quant_g32(_p(rows), rows.shape[0], I, _p(xq), _p(xs), _p(xsum)))
    return xq, xs, xsum


def dot_i8i8(w, x):
    """moty_hw_dot_i8i8 for every row of w [nrows][n] against x [n]."""
    w = np.ascontiguousarray(w, np.int8); x = np.ascontiguousarray(x, np.int8)
    w2 = w.reshape(-1, x.size) if x.size else w.reshape(w.shape[0] if w.ndim > 1 else 1, 0)
    out = np.empty(w2.shape[0], np.int32)
    _ck(lib().moty_cuda_dot_i8i8(_p(w2), _p(x), w2.shape[0], x.size, _p(out)))
    return out


def dot_i4i8(w4, x, nrows):
    w4 = np.ascontiguousarray(w4, np.uint8); x = np.ascontiguousarray(x, np.int8)
    out = np.empty(nrows, np.int32)
    _ck(lib().moty_cuda_dot_i4i8(_p(w4), _p(x), nrows, x.size, _p(out)))
    return out


def moe_topk(probs, K, norm_topk):
    """moty_moe_topk per row of already soft-maxed values."""
    p = _f32(probs); rows = p.reshape(-1, p.shape[-1])
    idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
    _ck(lib().moty_cuda_moe_topk(_p(rows), rows.shape[0], rows.shape[1], K, _p(idx), _p(w), int(norm_topk)))
    return idx, w


def route_topk(logits, K, want_probs=False):
    """route_topk (nn/moe.c:27-30): softmax + top-K with renormalisation."""
    lg = _f32(logits); rows = lg.reshape(-1, lg.shape[-1])
    idx = np.empty((rows.shape[0], K), np.int32); w = np.empty((rows.shape[0], K), np.float32)
    probs = np.empty(rows.shape, np.float32) if want_probs else None
    _ck(lib().moty_cuda_route_topk(_p(rows), rows.shape[0], rows.shape[1], K, _p(idx), _p(w), _p(probs)))
    return (idx, w, probs) if want_probs else (idx, w)


def argmax(v) -> int:
    """moty_argmax_v: first index of the maximum."""
    v = _f32(v).ravel()
    out = C.c_int(0)
    _ck(lib().moty_cuda_argmax(_p(v), v.size, C.byref(out)))
    return out.value


def head_argmax(head: "Mat", x, want_logits=False):
    """lm_head + greedy pick in one call (nn/head.c:134-135 then nn/sample.c:9-13): ids [S], optionally the logits."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None]
    S = x.shape[0]
    ids = np.empty(S, np.int32)
    lg = np.empty((S, head.O), np.float32) if want_logits else None
    _ck(lib().moty_cuda_head_argmax(head.h, _p(x), S, _p(ids), _p(lg) if want_logits else None))
    return (ids, lg) if want_logits else ids


class Attn:
    """The attention core of one layer with its KV cache on a GPU (nn/attn.c:29-74 without the projections):
    ``core(q, k, v, pos_base)`` norms and rotates q and k, stores k and v at their positions and returns ctx."""

    def __init__(self, H, KV, hd, max_t, theta=1e6, eps=1e-6, rot=None, qn=None, kn=None, kv8=False, device=0,
                 gemma=False, window=0, scale=0.0, vn=None):
        self.H, self.KV, self.hd, self.max_t = H, KV, hd, max_t
        h = C.c_void_p()
        qn = None if qn is None else _f32(qn); kn = None if kn is None else _f32(kn)
        if gemma:
            # engines/gemma.c's attention: qn / kn / vn are the norm MULTIPLIERS (1 + w), rot = rotated pairs of the p-RoPE
            vn = None if vn is None else _f32(vn)
            _ck(lib().moty_cuda_attn_create_gemma(C.byref(h), H, KV, hd, hd // 2 if rot is None else rot, C.c_float(theta), C.c_float(eps),
                                                  _p(qn) if qn is not None else None, _p(kn) if kn is not None else None,
                                                  _p(vn) if vn is not None else None, int(window), C.c_float(scale),
                                                  max_t, 1 if kv8 else 0, device))
        else:
            _ck(lib().moty_cuda_attn_create(C.byref(h), H, KV, hd, hd if rot is None else rot, C.c_float(theta), C.c_float(eps),
                                            _p(qn) if qn is not None else None, _p(kn) if kn is not None else None,
                                            max_t, 1 if kv8 else 0, device))
        self.h = h

    def core(self, q, k, v, pos_base):
        q = _f32(q); k = _f32(k); v = _f32(v); S = q.shape[0]
        ctx = np.empty((S, self.H * self.hd), np.float32)
        _ck(lib().moty_cuda_attn_core(self.h, _p(ctx), _p(q), _p(k), _p(v), S, pos_base))
        return ctx

    def core_dev(self, ctx_ptr, q_ptr, k_ptr, v_ptr, S, pos_base, stream=0):
        _ck(lib().moty_cuda_attn_core_dev(self.h, C.c_void_p(ctx_ptr), C.c_void_p(q_ptr), C.c_void_p(k_ptr), C.c_void_p(v_ptr),
                                          S, pos_base, C.c_void_p(stream)))

    def core_posdev(self, ctx_ptr, q_ptr, k_ptr, v_ptr, S, pos_dev_ptr, pos_max, stream=0):
        """The same with the first position read from a device int32 (for CUDA graph replay); pos_max bounds it.  With
        S = 1 the whole core is one scores launch (plus the merge) and q, k are NOT written back."""
        _ck(lib().moty_cuda_attn_core_posdev(self.h, C.c_void_p(ctx_ptr), C.c_void_p(q_ptr), C.c_void_p(k_ptr), C.c_void_p(v_ptr),
                                             S, C.c_void_p(pos_dev_ptr), pos_max, C.c_void_p(stream)))

    def gate_dev(self, ctx_ptr, gate_ptr, S, stream=0):
        """ctx *= sigmoid(gate) (moty_nn_attention_gated's last step), both [S][H*hd] on the device."""
        _ck(lib().moty_cuda_attn_gate_dev(self.h, C.c_void_p(ctx_ptr), C.c_void_p(gate_ptr), S, C.c_void_p(stream)))

    def close(self):
        if self.h:
            lib().moty_cuda_attn_free(self.h); self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_rows(w):
    """moty_quantize_rows (bits=8) computed on the GPU."""
    w = _f32(w); O, I = w.shape
    q = np.empty((O, I), np.int8); s = np.empty(O, np.float32)
    _ck(lib().moty_cuda_quantize_rows(_p(w), _p(q), _p(s), O, I))
    return q, s


def pack_q4r4(w):
    """moty_pack_q4r4_block over a whole matrix, computed on the GPU."""
    w = _f32(w); O, I = w.shape
    nblk, nb = (O + 3) // 4, I // 32
    q4 = np.empty(nblk * nb * 64, np.uint8); s16 = np.empty(nblk * nb * 4, np.uint16)
    _ck(lib().moty_cuda_pack_q4r4(_p(w), O, I, _p(q4), _p(s16)))
    return q4, s16


# ---------------------------------------------------------------------------
# blocks
# ---------------------------------------------------------------------------
def dense_ffn(gate: Mat, up: Mat, down: Mat, x, act: int = ACT_SILU):
    """moty_nn_dense_ffn / the engines' mlp(): down(act(gate x) * up x)."""
    x = _f32(x)
    if x.ndim == 1:
        x = x[None, :]
    out = np.empty((x.shape[0], down.O), np.float32)
    _ck(lib().moty_cuda_ffn(gate.h, up.h, down.h, act, _p(out), _p(x), x.shape[0]))
    return out


def dense_ffn_dev(gate: Mat, up: Mat, down: Mat, out_ptr: int, x_ptr: int, S: int, act: int = ACT_SILU, stream: int = 0):
    _ck(lib().moty_cuda_ffn_dev(gate.h, up.h, down.h, act, C.c_void_p(out_ptr), C.c_void_p(x_ptr), S, C.c_void_p(stream)))


class Moe:
    """One MoE layer with its experts resident on a GPU (the device-side
    MotyMoeView + ExpertCache).  ``e_lo:e_hi`` is this GPU's expert shard."""

    def __init__(self, E, K, I, D, efmt=WF_I8, e_lo=0, e_hi=None, device=0):
        self.E, self.K, self.I, self.D, self.efmt, self.device = E, K, I, D, efmt, device
        self.e_lo, self.e_hi = e_lo, E if e_hi is None else e_hi
        h = C.c_void_p()
        _ck(lib().moty_cuda_moe_create(C.byref(h), E, K, I, D, efmt, self.e_lo, self.e_hi, device))
        self.h = h
        self.router = None

    def upload_expert(self, eid, g, gs, u, us, d, ds):
        arrs = [np.ascontiguousarray(a) for a in (g, gs, u, us, d, ds)]
        _ck(lib().moty_cuda_moe_upload_expert(self.h, eid, *(_p(a) for a in arrs)))

    def upload_expert_i4(self, eid, g4, gs, u4, us, d4, ds):
        """LFM2's int4 expert rows (nibble rows + f32 row scales); the layer must hold MOTY_WF_I8 experts."""
        a4 = [np.ascontiguousarray(a, np.uint8) for a in (g4, u4, d4)]
        sc = [np.ascontiguousarray(a, np.float32) for a in (gs, us, ds)]
        _ck(lib().moty_cuda_moe_upload_expert_i4(self.h, eid, _p(a4[0]), _p(sc[0]), _p(a4[1]), _p(sc[1]), _p(a4[2]), _p(sc[2])))

    def set_sigmoid_gate(self, on: bool = True, expert_bias=None):
        """LFM2's gate (sigmoid + expert bias, nn/moe.c:10-25) instead of softmax + top-K."""
        b = None if expert_bias is None else np.ascontiguousarray(expert_bias, np.float32)
        _ck(lib().moty_cuda_moe_set_sigmoid_gate(self.h, int(bool(on)), _p(b)))

    def set_router(self, router: Mat | None):
        self.router = router
        _ck(lib().moty_cuda_moe_set_router(self.h, router.h if router else None))

    def d1(self, x, logits=None):
        """moty_nn_moe_topk_d1: one token."""
        x = _f32(x).reshape(1, self.D); out = np.empty((1, self.D), np.float32)
        lg = None if logits is None else _f32(logits).reshape(1, self.E)
        _ck(lib().moty_cuda_moe_d1(self.h, _p(out), _p(x), _p(lg)))
        return out

    def batch(self, x, logits=None):
        """moty_nn_moe_topk_batch: S tokens, experts in ascending id."""
        x = _f32(x).reshape(-1, self.D); S = x.shape[0]; out = np.empty((S, self.D), np.float32)
        lg = None if logits is None else _f32(logits).reshape(S, self.E)
        _ck(lib().moty_cuda_moe_batch(self.h, _p(out), _p(x), S, _p(lg)))
        return out

    def olmoe(self, x, logits=None, norm_topk=0):
        """engines/olmoe.c moe(): per token, selection order."""
        x = _f32(x).reshape(-1, self.D); S = x.shape[0]; out = np.empty((S, self.D), np.float32)
        lg = None if logits is None else _f32(logits).reshape(S, self.E)
        _ck(lib().moty_cuda_olmoe_moe(self.h, _p(out), _p(x), S, _p(lg), int(norm_topk)))
        return out

    def apply_dev(self, out_ptr, x_ptr, S, logits_ptr=0, order=0, norm_topk=1, idx_ptr=0, w_ptr=0, stream=0):
        _ck(lib().moty_cuda_moe_apply_dev(self.h, C.c_void_p(out_ptr), C.c_void_p(x_ptr), S,
                                          C.c_void_p(logits_ptr), order, norm_topk,
                                          C.c_void_p(idx_ptr), C.c_void_p(w_ptr), C.c_void_p(stream)))

    def free(self):
        if self.h:
            lib().moty_cuda_moe_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def q8_apply_noalloc(y_ptr: int, x_ptr: int, q_ptr: int, scale_ptr: int, S: int, I: int, O: int,
                     device: int = 0, stream: int = 0) -> None:
    """The Q8_0 product for hosts that must not allocate: device pointers in and
    out, scratch in a fixed array inside the library (S <= 8, I <= 16384)."""
    _ck(lib().moty_cuda_q8_apply_noalloc(C.c_void_p(y_ptr), C.c_void_p(x_ptr), C.c_void_p(q_ptr), C.c_void_p(scale_ptr),
                                         S, I, O, device, C.c_void_p(stream)))
