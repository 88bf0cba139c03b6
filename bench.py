#!/usr/bin/env python
"""Benchmark of the Q8_0 decode GEMV path (the op-level sweep of the baseline).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of the S=1 Q8_0 GEMV over the six sweep shapes (O x I:
1024x1024, 3072x1024, 1024x3072, 151936x1024, 15360x3840, 3840x15360; int8
weights U[-127,127], f32 row scales U(0.001,0.02), activations N(0,1), seed 0).
The weights of one pass total 280 MB, more than the 126 MB L2, so every pass
streams from HBM.

value      algorithmic GB/s with activations and results resident on the GPU
           (moty_cuda_mat_apply_dev): K passes replayed from CUDA graphs, nothing but the
           passes' launches between the two events on the launch stream, max over ranks
e2e        the same passes through the host-pointer entry moty_cuda_mat_apply
           (pinned host buffers; H2D of x and D2H of y inside the timed region)
roofline   the dominant kernel -- the launch that holds the 151936x1024 matrix: by default the
           one launch of the whole pass (q8_multi_kernel, six matrices), with --multi-max-mb 64
           or --no-multi that matrix's own GEMV --: bytes / its own average launch time,
           measured with events around its launch in K further passes right after the timed region
cpu_baseline / --impl reference
           the reference's own OpenMP code (oracle/_ref, else the C restatement)
           on the host cores, same passes

N > 1: one process per GPU (torchrun), independent replicas of the sweep, no
data-path collective (the op sweep does not shard); value = N passes / max time.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(1024, 1024), (3072, 1024), (1024, 3072), (151936, 1024), (15360, 3840), (3840, 15360)]
DOMINANT = 3                                   # index of the 151936x1024 matrix
METRIC = "Q8_0 GEMV HBM GB/s (op-level sweep, S=1 decode)"
WORKLOAD = "configs[1]: op-level Q8_0 sweep, six shapes, S=1, seed 0"


def config_dict(world):
    """The workload description both arms print (the GPU arm and --impl reference), key for key."""
    return {"workload": WORKLOAD, "l2": "inputs_larger_than_l2 (280 MB of weights per pass, L2 126 MB)",
            "parallelism": "replicas" if world > 1 else "single", "bytes_per_step": sum(algo_bytes(*s) for s in SHAPES)}


def algo_bytes(O, I, S=1):
    """Q8_0 bytes per call: weights + row scales + activations in + results out."""
    return O * I + 4 * O + 4 * S * I + 4 * S * O


def make_inputs(seed=0):
    rng = np.random.default_rng(seed)
    mats = []
    for (O, I) in SHAPES:
        W = rng.integers(-127, 128, size=(O, I), dtype=np.int8)
        sc = rng.uniform(0.001, 0.02, O).astype(np.float32)
        x = rng.standard_normal((1, I)).astype(np.float32)
        mats.append((W, sc, x))
    return mats


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def profile_traffic(name="q8_stream_gemv_151936x1024.md"):
    """DRAM bytes per launch of the dominant kernel, from the committed ncu summary."""
    p = os.path.join(ROOT, "profiles", name)
    if os.path.exists(p):
        m = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", open(p).read())
        if m:
            return float(m.group(1))
    return None


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksThrottleReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksThrottleReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksThrottleReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksThrottleReasonSwPowerCap}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# CPU arm: the reference's own code on the host cores
# ---------------------------------------------------------------------------
def cpu_arm(mats, steps, warmup, budget_s=None):
    """Time passes of the sweep with moty_matmul_q_s.  Returns (GB/s, cores, kind, passes, seconds)."""
    from oracle import Oracle, Ref
    if Ref.available():
        r = Ref(); kind = "reference"
        # all the host threads this process may use (a launcher may have put OMP_NUM_THREADS=1 in
        # the environment for its ranks; rank 0 alone runs this arm)
        avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        r.set_threads(avail)
        cores = r.threads()
        call = r.matmul_q_s
    else:
        r = Oracle(); kind = "port"; cores = os.cpu_count() or 1
        call = r.matmul_q_s
    for _ in range(max(warmup, 1)):
        for (W, sc, x) in mats:
            call(x, W, sc)
    total = sum(algo_bytes(*s) for s in SHAPES)
    t0 = time.perf_counter(); done = 0
    while done < steps:
        for (W, sc, x) in mats:
            call(x, W, sc)
        done += 1
        if budget_s is not None and time.perf_counter() - t0 > budget_s and done >= 3:
            break
    dt = time.perf_counter() - t0
    return total * done / dt / 1e9, cores, kind, done, dt


def decode_summary(extras):
    """The 'decode tok/s' half of the metric's name, lifted out of the extras: the Qwen3-0.6B-shaped greedy decode through
    the device-resident entries (python-driven and as a replayed CUDA graph) and the reference's engine beside it."""
    if not extras or "decode_qwen3_0.6b" not in extras:
        return None
    d, e = extras.get("decode_qwen3_0.6b") or {}, extras.get("engine_qwen3_0.6b") or {}
    return {"config": "configs[0] shape (Qwen3-0.6B), int8, batch 1, 64-token prompt",
            "gpu_device_resident_graph": d.get("graph_decode_tok_s"), "gpu_device_resident_python": d.get("decode_tok_s"),
            "reference_engine_cpu": (e.get("cpu_reference") or {}).get("decode_tok_s"),
            "reference_engine_gpu_hook": (e.get("gpu_through_mat_apply_hook") or {}).get("decode_tok_s"),
            "reference_engine_gpu_device_resident_step": (e.get("gpu_device_resident_step") or {}).get("decode_tok_s"),
            "hbm_ceiling_tok_s": round(measured_peak()[0] * 1e9 / 598.0e6, 0)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    mats = make_inputs()
    gbs, cores, kind, done, dt = cpu_arm(mats, args.steps, args.warmup, budget_s=120.0)
    line = {"impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s", "n_gpus": args.gpus,
            "steps": done, "warmup": args.warmup, "ms_per_step": round(dt / done * 1e3, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8xint8->int32",
            "data": "synthetic", "config": config_dict(int(os.environ.get("WORLD_SIZE", "1"))),
            "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
                             "sample": f"{done} passes of the sweep, {dt:.1f} s"},
            "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
# extras: the other rows of the op-level sweep, timed per shape (reported beside the
# headline, not part of it): Q8_0 at S=16 and S=512, Q4R4 at S=1, 16 and 512, and one
# library int8 GEMM as the calibration point for the int8 tensor peak
# ---------------------------------------------------------------------------
def q4r4_bytes(O, I, S=1):
    return (O + 3) // 4 * (I // 32) * 72 + 4 * S * I + 4 * S * O


def run_extras(torch, mb, dev, stream, W8, local):
    sp = stream.cuda_stream
    out = {"rows": []}
    a = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=dev)
    b = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=dev)
    best = 1e9
    for _ in range(8):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); torch._int_mm(a, b); e1.record(); torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    out["int8_library_gemm_8192_tops"] = round(2 * 8192 ** 3 / (best * 1e-3) / 1e12, 1)
    del a, b
    rng = np.random.default_rng(1)
    W4 = []
    for (O, I) in SHAPES:
        nblk, nb = (O + 3) // 4, I // 32
        q4 = rng.integers(0, 256, nblk * nb * 64, dtype=np.uint8)
        s16 = np.full(nblk * nb * 4, 0x1A00, np.uint16)               # f16 0.00293
        W4.append(mb.Mat.q4r4(q4, s16, O, I, device=local))
    Wg = []                                                            # the legacy grouped int4 (row-major nibbles, f32 group scales)
    for (O, I) in SHAPES:
        Wg.append(mb.Mat.i4g(rng.integers(0, 256, (O, I // 2), dtype=np.uint8),
                             np.full((O, I // 32), 0.003, np.float32), O, I, device=local))
    with torch.cuda.stream(stream):
        for fmt, mats, S, passes in (("q8_0", W8, 16, 6), ("q8_0", W8, 512, 3), ("q4r4", W4, 1, 10), ("q4r4", W4, 16, 4), ("q4r4", W4, 512, 2),
                                       ("q4r4_relaxed", W4, 16, 4), ("q4r4_relaxed", W4, 512, 2), ("i4g", Wg, 16, 4), ("i4g", Wg, 512, 2)):
            # (q4r4_relaxed: after moty_cuda_set_q4r4_batch_relaxed(1) -- one formula for a group's term, within 1e-5)
            mb.lib().moty_cuda_set_q4r4_batch_relaxed(1 if fmt == "q4r4_relaxed" else 0)
            xs = [torch.randn((S, I), device=dev) for (_, I) in SHAPES]
            ys = [torch.empty((S, O), device=dev) for (O, _) in SHAPES]
            ev = [[] for _ in SHAPES]
            for p in range(passes + 1):
                for i, (w, x, y) in enumerate(zip(mats, xs, ys)):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    mb.mat_apply_dev(w, y.data_ptr(), x.data_ptr(), S, sp)
                    e1.record(stream)
                    if p > 0:
                        ev[i].append((e0, e1))
            torch.cuda.synchronize()
            for i, (O, I) in enumerate(SHAPES):
                us = statistics.mean(a.elapsed_time(b) for a, b in ev[i]) * 1e3
                nbytes = (algo_bytes(O, I, S) if fmt == "q8_0" else
                          O * I // 2 + 4 * O * (I // 32) + 4 * S * I + 4 * S * O if fmt == "i4g" else q4r4_bytes(O, I, S))
                out["rows"].append({"fmt": fmt, "S": S, "O": O, "I": I, "us": round(us, 2),
                                    "GBs": round(nbytes / us / 1e3, 1), "TOPS": round(2.0 * S * O * I / us / 1e6, 2)})
            del xs, ys
    mb.lib().moty_cuda_set_q4r4_batch_relaxed(0)
    del W4, Wg
    out["moe"] = run_moe_extras(torch, mb, dev, stream, local)
    out["blocks"] = run_block_extras(torch, mb, dev, stream, local)
    # the model-level view of the same kernels: a greedy decode of the configs[0] shape (wall clock, whole steps)
    try:
        out["decode_qwen3_0.6b"] = run_decode_qwen(torch, mb, np.random.default_rng(3), 64, local)
    except Exception as e:                              # an extra must not cost the headline line
        out["decode_qwen3_0.6b"] = {"error": str(e)[:200]}
    try:
        out["engine_qwen3_0.6b"] = run_engine_qwen()
    except Exception as e:
        out["engine_qwen3_0.6b"] = {"error": str(e)[:200]}
    return out


def run_engine_qwen(ngen=128):
    """The reference's own `qwen` engine on the Qwen3-0.6B-shaped synthetic snapshot (64-token prompt, ngen greedy
    steps, QBITS=8): once as it is on the host cores, once with every matrix attached to the GPU through the
    reference-side shim (moty_b200/shim/hw_cuda.c: the per-matrix moty_mat_apply hook, host pointers, a copy in and
    out per call).  Reports the engine's prefill / decode tok/s of both runs and whether ids and logit rows agree.  The
    decode figure is the time in step() + argmax per token, as in the engine's own loop (runtime/rt_gen_loop.h:46-84);
    writing the trace rows (a hash of every 600 KB logit row) is the shim's instrument and is timed apart, in all three runs."""
    import re
    import shutil
    import tempfile
    from moty_b200 import shim
    from moty_b200.shim.make_snapshot import write_snapshot
    if shim.engine_binary() is None:
        return {"unavailable": "the shimmed engine is not built here (needs the reference checkout at build time)"}
    tmp = tempfile.mkdtemp(prefix="moty_snap_")
    try:
        write_snapshot(tmp, prompt=64, gen=ngen)
        out = {}
        traces = {}
        for name, cuda in (("cpu_reference", 0), ("gpu_through_mat_apply_hook", 1), ("gpu_device_resident_step", 2)):
            tr = os.path.join(tmp, f"trace_{int(cuda)}.txt")
            r = shim.run_engine(tmp, cuda=cuda, trace=tr, timeout=600)
            if r.returncode != 0:
                return {"error": (r.stderr or r.stdout)[-300:]}
            m = re.search(r"prefill (\d+) tok [\d.]+ s ([\d.]+) tok/s \| decode (\d+) tok [\d.]+ s ([\d.]+) tok/s", r.stdout)
            out[name] = {"prefill_tok_s": float(m.group(2)), "decode_tok_s": float(m.group(4))}
            traces[cuda] = open(tr).read()
        ids_of = lambda t: [ln.split()[1] for ln in t.splitlines()]
        out["hook_ids_and_logit_rows_identical_to_cpu"] = traces[0] == traces[1]
        a, b = ids_of(traces[0]), ids_of(traces[2])
        first = next((i for i, (u, v) in enumerate(zip(a, b)) if u != v), len(a))
        out["device_resident_free_running_ids_equal_to_cpu_for_steps"] = first      # (attention sums in another order: see tests/test_engine_shim.py)
        out["host_threads"] = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
        out["workload"] = f"Qwen3-0.6B shape, QBITS=8, 64-token prompt + {ngen} greedy steps, REF= mode of the reference's qwen engine"
        return out
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


def run_decode_qwen(torch, mb, rng, ngen, device, fold=None):
    """A whole greedy decode of the configs[0] shape (Qwen3-0.6B: 28 layers, hidden 1024, 16/8 heads of 128, FFN 3072,
    vocabulary 151936, tied int8 head) on synthetic int8 weights: a 64-token prompt, then ngen tokens launched entry by
    entry from Python, then the same tokens as a replayed CUDA graph of one decode step."""
    import time
    from moty_b200.decoder import DenseDecoder, DenseLayer
    NL, D, H, KV, hd, I, V, PROMPT = 28, 1024, 16, 8, 128, 3072, 151936, 64
    raw = lambda O, K: (rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.0002, 0.0006, O).astype(np.float32))
    mk = lambda O, K: mb.Mat.i8(*raw(O, K), device=device)
    one = lambda n: np.ones(n, np.float32)
    def layer():
        q, k, v = raw(H * hd, D), raw(KV * hd, D), raw(KV * hd, D)
        qkv = mb.Mat.i8(np.concatenate([q[0], k[0], v[0]]), np.concatenate([q[1], k[1], v[1]]), device=device)
        return DenseLayer(mb.Mat.i8(*q, device=device), mb.Mat.i8(*k, device=device), mb.Mat.i8(*v, device=device), mk(D, H * hd),
                          mk(I, D), mk(I, D), mk(D, I), one(D), one(D), one(hd), one(hd), qkv=qkv)
    layers = [layer() for _ in range(NL)]
    head = mb.Mat.i8(rng.integers(-127, 128, (V, D), dtype=np.int8), rng.uniform(0.005, 0.015, V).astype(np.float32), device=device)
    dec = DenseDecoder(layers, head, one(D), H, KV, hd, PROMPT + ngen + 8, max_S=PROMPT, device=device, fold_addnorm=fold)
    prompt = np.random.default_rng(1).integers(0, V, PROMPT).astype(np.int32)
    dec.step(prompt, 0); dec.step([1], PROMPT)                       # warm-up (allocations, attributes)
    torch.cuda.synchronize(); t0 = time.perf_counter()
    tok = dec.step(prompt, 0)
    torch.cuda.synchronize(); t1 = time.perf_counter()
    toks = [tok]
    for i in range(ngen):
        toks.append(dec.step([toks[-1]], PROMPT + i))
    torch.cuda.synchronize(); t2 = time.perf_counter()
    tg = dec.greedy_graph(tok, PROMPT, ngen)                          # captures on first use
    torch.cuda.synchronize(); t3 = time.perf_counter()
    tg = dec.greedy_graph(tok, PROMPT, ngen)
    torch.cuda.synchronize(); t4 = time.perf_counter()
    wbytes = sum(m.nbytes() for l in layers for m in (l.qkv, l.o, l.gate, l.up, l.down)) + head.nbytes()
    res = {"prefill_tok_s": round(PROMPT / (t1 - t0), 1), "decode_tok_s": round(ngen / (t2 - t1), 1),
           "ms_per_token": round((t2 - t1) / ngen * 1e3, 3), "weight_MB_per_token": round(wbytes / 1e6, 1),
           "GBs": round(wbytes * ngen / (t2 - t1) / 1e9, 1), "launch": "python-driven device entries, no graph",
           "graph_decode_tok_s": round(ngen / (t4 - t3), 1), "graph_ms_per_token": round((t4 - t3) / ngen * 1e3, 3),
           "graph_GBs": round(wbytes * ngen / (t4 - t3) / 1e9, 1), "graph_equals_direct": tg == toks[1:]}
    dec.close()
    for l in layers:
        for m in (l.q, l.k, l.v, l.o, l.gate, l.up, l.down, l.qkv):
            m.free()
    head.free()
    return res


def run_block_extras(torch, mb, dev, stream, local):
    """The callers either side of the matmuls, one decode token: a dense int8 SiLU FFN block (Qwen3-0.6B shape) and the
    attention core against a 4096-position f32 cache (16 heads, 8 KV heads, head_dim 128); CUDA events over 50 calls."""
    rng = np.random.default_rng(5)
    res = {}
    sp = stream.cuda_stream
    def timed(fn, n=50):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) * 1e3 / n, 2)
    with torch.cuda.stream(stream):
        D, I = 1024, 3072
        mk = lambda O, K: mb.Mat.i8(rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32), device=local)
        G, U, Dn = mk(I, D), mk(I, D), mk(D, I)
        x = torch.randn((1, D), device=dev); y = torch.empty((1, D), device=dev)
        res["ffn_decode_1024x3072_us"] = timed(lambda: mb.dense_ffn_dev(G, U, Dn, y.data_ptr(), x.data_ptr(), 1, stream=sp))
        del G, U, Dn
        H, KV, hd, POS = 16, 8, 128, 4096
        a = mb.Attn(H, KV, hd, POS + 1, qn=np.ones(hd, np.float32), kn=np.ones(hd, np.float32), device=local)
        q = torch.randn((1, H * hd), device=dev); k = torch.randn((1, KV * hd), device=dev); v = torch.randn((1, KV * hd), device=dev)
        ctx = torch.empty((1, H * hd), device=dev)
        res["attn_decode_pos4096_us"] = timed(lambda: a.core_dev(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, POS, stream=sp))
        a.close()
    return res


MOE_SHAPES = {"olmoe": (64, 8, 1024, 2048, "i8"), "qwen3-30b-a3b": (128, 8, 768, 2048, "q4r4")}


def make_moe_layers(mb, name, nlayers, local, rng):
    """nlayers routed layers of the named shape with different random experts, GPU-resident."""
    E, K, I, D, f = MOE_SHAPES[name]
    fmt = mb.WF_I8 if f == "i8" else mb.WF_Q4R4
    layers = []
    for _ in range(nlayers):
        m = mb.Moe(E, K, I, D, efmt=fmt, device=local)
        for e in range(E):
            if fmt == mb.WF_I8:
                g = rng.integers(-127, 128, (I, D), dtype=np.int8); u = rng.integers(-127, 128, (I, D), dtype=np.int8)
                d = rng.integers(-127, 128, (D, I), dtype=np.int8)
                gs = rng.uniform(0.001, 0.02, I).astype(np.float32); us = rng.uniform(0.001, 0.02, I).astype(np.float32)
                ds = rng.uniform(0.001, 0.02, D).astype(np.float32)
            else:
                ng, nd = (I // 4) * (D // 32), (D // 4) * (I // 32)
                g = rng.integers(0, 256, ng * 64, dtype=np.uint8); u = rng.integers(0, 256, ng * 64, dtype=np.uint8)
                d = rng.integers(0, 256, nd * 64, dtype=np.uint8)
                gs = np.full(ng * 4, 0x1A00, np.uint16); us = np.full(ng * 4, 0x1A00, np.uint16); ds = np.full(nd * 4, 0x1A00, np.uint16)
            m.upload_expert(e, g, gs, u, us, d, ds)
        layers.append(m)
    per_expert = (3 * I * D + 4 * (2 * I + D)) if fmt == mb.WF_I8 else (2 * (I // 4) * (D // 32) * 72 + (D // 4) * (I // 32) * 72)
    return layers, per_expert


def time_moe(torch, layers, name, S, dev, stream, reps=5, run=16):
    """Microseconds per layer call: runs of `run` consecutive calls (a decode step runs its layers back
    to back), the weight sets cycled so that a layer's experts are not L2-resident when it runs."""
    E, K, I, D, _ = MOE_SHAPES[name]
    sp = stream.cuda_stream
    x = torch.randn((S, D), device=dev)
    logits = [torch.randn((S, E), device=dev) for _ in range(8)]
    outp = torch.empty((S, D), device=dev)
    order = 0 if S == 1 else 1

    def call(it):
        layers[it % len(layers)].apply_dev(outp.data_ptr(), x.data_ptr(), S, logits[it % 8].data_ptr(), order, 1, 0, 0, sp)
    for it in range(8):
        call(it)
    ev = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for it in range(run):
            call(it)
        e1.record(stream)
        ev.append((e0, e1))
    torch.cuda.synchronize()
    return statistics.mean(a.elapsed_time(b) for a, b in ev) * 1e3 / run


def run_moe_extras(torch, mb, dev, stream, local):
    """One routed MoE layer on the two MoE shapes of the baseline: OLMoE-1B-7B (E=64, K=8, expert FFN 1024, hidden
    2048, int8 experts) and Qwen3-30B-A3B (E=128, K=8, expert FFN 768, hidden 2048, Q4R4 experts): decode (S=1), a small
    batch (S=64) and the prefill sizes of the configs (OLMoE: its 512-token prompt; Qwen3-30B-A3B: 1024 tokens of its
    8 x 1024).  Bytes = the touched experts' gate+up+down (codes and scales); ops = 2 * S * K * 3 * I * D."""
    rng = np.random.default_rng(2)
    rows = []
    for name in MOE_SHAPES:
        E, K, I, D, f = MOE_SHAPES[name]
        layers, per_expert = make_moe_layers(mb, name, 4, local, rng)
        with torch.cuda.stream(stream):
            for S in (1, 64, 512 if f == "i8" else 1024):
                us = time_moe(torch, layers, name, S, dev, stream, reps=5 if S <= 64 else 3, run=16 if S <= 64 else 4)
                touched = K * per_expert if S == 1 else min(E, S * K) * per_expert
                row = {"layer": name, "S": S, "us": round(us, 1), "expert_GBs": round(touched / us / 1e3, 1),
                       "TOPS": round(2.0 * S * K * 3 * I * D / us / 1e6, 1)}
                if f == "i8" and S >= 64:
                    prev = mb.lib().moty_cuda_set_moe_batch_path(0)
                    row["us_mma_sync_tiles"] = round(time_moe(torch, layers, name, S, dev, stream, reps=3, run=4), 1)
                    mb.lib().moty_cuda_set_moe_batch_path(prev)
                    row["path"] = "tcgen05 grouped (gate+up+SiLU one pass), 7 launches"
                if f == "q4r4" and S >= 64:             # the grouped products with one formula per group term (opt-in, within 1e-5)
                    prev = mb.lib().moty_cuda_set_q4r4_batch_relaxed(1)
                    row["us_relaxed"] = round(time_moe(torch, layers, name, S, dev, stream, reps=3, run=4), 1)
                    mb.lib().moty_cuda_set_q4r4_batch_relaxed(prev)
                rows.append(row)
        for m in layers:
            m.free()
    return rows


# ---------------------------------------------------------------------------
# N > 1: the sharded forms of the path, timed beside the replicas of the headline sweep.
# Expert-parallel routed layers of the two MoE shapes (experts in contiguous ranges per rank) and the
# row-sharded decode products of the Gemma-4-12B shape with their all-gather.  Every time is CUDA events
# around a run of calls on the rank's stream, max over ranks; rank 0 also runs the unsharded layer or
# matrix on its own GPU for the same tokens, so efficiency = t(1 GPU) / (N * t(N GPUs)).
# ---------------------------------------------------------------------------
def _pool_expert(mb, name, rng):
    E, K, I, D, f = MOE_SHAPES[name]
    if f == "i8":
        return (rng.integers(-127, 128, (I, D), dtype=np.int8), rng.uniform(0.001, 0.02, I).astype(np.float32),
                rng.integers(-127, 128, (I, D), dtype=np.int8), rng.uniform(0.001, 0.02, I).astype(np.float32),
                rng.integers(-127, 128, (D, I), dtype=np.int8), rng.uniform(0.001, 0.02, D).astype(np.float32))
    ng, nd = (I // 4) * (D // 32), (D // 4) * (I // 32)
    return (rng.integers(0, 256, ng * 64, dtype=np.uint8), np.full(ng * 4, 0x1A00, np.uint16),
            rng.integers(0, 256, ng * 64, dtype=np.uint8), np.full(ng * 4, 0x1A00, np.uint16),
            rng.integers(0, 256, nd * 64, dtype=np.uint8), np.full(nd * 4, 0x1A00, np.uint16))


def run_sharded(torch, dist, mb, dev, local, rank, world, steps):
    from moty_b200.parallel import ExpertParallelMoe, RowShardedMat, shard_rows
    rows = []
    gen = torch.Generator().manual_seed(11)
    use_graph = os.environ.get("MOTY_BENCH_SHARDED_GRAPH", "0") == "1"     # capturing the collectives failed on this stack (capture invalidated): off

    def timed(fn, n):
        for _ in range(9):                                     # more than the weight sets that fn cycles through: every set's
            fn()                                               # buffers, communicator paths and peer mappings exist before timing
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_local(fn, n):
        for _ in range(9):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / n

    def timed_graph(fn, collective, per_graph=16, replays=10):
        """Decode-sized calls are host-bound when launched one by one from Python (a collective costs ~20 us of
        dispatcher time): capture per_graph calls into one CUDA graph (NCCL collectives are capturable) and time replays."""
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            # thread_local: the communication library's watchdog thread queries events while this thread captures
            with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                for _ in range(per_graph):
                    fn()
            g.replay(); side.synchronize()
            if collective:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for _ in range(replays):
                g.replay()
            e1.record(side); side.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / (replays * per_graph)
        if collective:
            t = torch.tensor([us], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            us = float(t.item())
        torch.cuda.current_stream().wait_stream(side)
        return us

    NL = 4                                                     # weight sets cycled so that a layer's experts are not L2-resident
    for name, prefill_tokens in (("olmoe", 512), ("qwen3-30b-a3b", 8192)):
        E, K, I, D, f = MOE_SHAPES[name]
        if E % world or prefill_tokens % world:
            continue
        fmt = mb.WF_I8 if f == "i8" else mb.WF_Q4R4
        rng = np.random.default_rng(21)
        pool = [_pool_expert(mb, name, rng) for _ in range(4)]
        eps = [ExpertParallelMoe(E, K, I, D, efmt=fmt, device=local) for _ in range(NL)]
        ones = [mb.Moe(E, K, I, D, efmt=fmt, device=local) for _ in range(NL)] if rank == 0 else []
        for li in range(NL):
            for e in range(E):
                ex = pool[(e + li) % 4]
                eps[li].upload_expert(e, *ex)
                if rank == 0:
                    ones[li].upload_expert(e, *ex)
        it = [0]
        # decode: the same token on every rank
        x1 = torch.randn((1, D), generator=gen).to(dev); l1 = [torch.randn((1, E), generator=gen).to(dev) for _ in range(8)]
        def ep_dec():
            it[0] += 1
            eps[it[0] % NL].decode(x1, l1[it[0] % 8])
        us_ep_eager = timed(ep_dec, max(steps, 50))
        us_ep = timed_graph(ep_dec, True) if use_graph else us_ep_eager
        us_one = None
        if rank == 0:
            o1 = torch.empty((1, D), device=dev)
            def one_dec():
                it[0] += 1
                ones[it[0] % NL].apply_dev(o1.data_ptr(), x1.data_ptr(), 1, l1[it[0] % 8].data_ptr(), 0, 1, 0, 0,
                                           mb.stream_handle(torch.cuda.current_stream()))
            us_one = timed_graph(one_dec, False) if use_graph else timed_local(one_dec, max(steps, 50))
        def ep_peer():
            it[0] += 1
            eps[it[0] % NL].decode_peer(x1, l1[it[0] % 8])
        us_peer = timed(ep_peer, max(steps, 50))
        rows.append({"layer": name, "mode": "expert-parallel decode, one token replicated, rows exchanged by the library's own kernels over NVLink peer memory (2 launches, no collective)",
                     "tokens": 1, "experts_per_gpu": E // world, "us_sharded": round(us_peer, 1), "us_one_gpu": us_one and round(us_one, 1),
                     "launch": "python, call by call"})
        rows.append({"layer": name, "mode": "expert-parallel decode, one token replicated, all-reduce of the [K][D] row table",
                     "tokens": 1, "experts_per_gpu": E // world, "us_sharded": round(us_ep, 1), "us_one_gpu": us_one and round(us_one, 1),
                     "launch": "16 layer calls per replayed CUDA graph" if use_graph else "python, call by call",
                     "us_sharded_eager_python": round(us_ep_eager, 1)})
        # prefill: the prompt's tokens split over the ranks, all-gather + partial sums + reduce-scatter
        s = prefill_tokens // world
        xs = torch.randn((s, D), generator=gen).to(dev); ls = torch.randn((s, E), generator=gen).to(dev)
        def ep_pre():
            it[0] += 1
            eps[it[0] % NL].forward_gathered(xs, ls, order=1)
        us_ep = timed(ep_pre, 5)
        us_one = None
        if rank == 0:
            xa = torch.randn((prefill_tokens, D), generator=gen).to(dev); la = torch.randn((prefill_tokens, E), generator=gen).to(dev)
            oa = torch.empty_like(xa)
            def one_pre():
                it[0] += 1
                ones[it[0] % NL].apply_dev(oa.data_ptr(), xa.data_ptr(), prefill_tokens, la.data_ptr(), 1, 1, 0, 0,
                                           mb.stream_handle(torch.cuda.current_stream()))
            us_one = timed_local(one_pre, 5)
            del xa, la, oa
        rows.append({"layer": name, "mode": "expert-parallel prefill, all-gather + partial sums + reduce-scatter",
                     "tokens": prefill_tokens, "experts_per_gpu": E // world, "us_sharded": round(us_ep, 1),
                     "us_one_gpu": us_one and round(us_one, 1)})
        for m in ones:
            m.free()
        for e_ in eps:
            e_.moe.free()
        del eps, ones
    # row-sharded decode products of the Gemma-4-12B shape: up/gate, down and the 262144-row tied head, one pass of
    # the three per call (more than L2 per GPU at every N), each followed by its all-gather
    rng = np.random.default_rng(22)
    shapes = [(15360, 3840), (3840, 15360), (262144, 3840)]
    sh, full, xs_ = [], [], []
    for (O, I) in shapes:
        lo, hi, per = shard_rows(O, world, rank, 1)
        # only this rank's rows are generated (timing does not depend on the values)
        wq = rng.integers(-127, 128, (hi - lo, I), dtype=np.int8); sc = np.full(hi - lo, 0.01, np.float32)
        sh.append(RowShardedMat.from_local_rows(mb.WF_I8, wq, sc, O, I, device=local))
        xs_.append(torch.randn((1, I), generator=gen).to(dev))
        if rank == 0:
            wf = rng.integers(-127, 128, (O, I), dtype=np.int8)
            full.append((mb.Mat.i8(wf, np.full(O, 0.01, np.float32), device=local), torch.empty((1, O), device=dev)))
            del wf
        del wq
    us_sh_eager = timed(lambda: [m.decode(x) for m, x in zip(sh, xs_)], max(steps, 30))
    one_pass = lambda: [mb.mat_apply_dev(w, y.data_ptr(), x.data_ptr(), 1, mb.stream_handle(torch.cuda.current_stream()))
                        for (w, y), x in zip(full, xs_)]
    us_sh = timed_graph(lambda: [m.decode(x) for m, x in zip(sh, xs_)], True, per_graph=4) if use_graph else us_sh_eager
    us_one = None
    if rank == 0:
        us_one = timed_graph(one_pass, False, per_graph=4) if use_graph else timed_local(one_pass, max(steps, 30))
    rows.append({"layer": "gemma-4-12b dense", "mode": "row-sharded decode: 15360x3840 + 3840x15360 + 262144x3840 head, all-gather after each",
                 "tokens": 1, "us_sharded": round(us_sh, 1), "us_one_gpu": us_one and round(us_one, 1),
                 "launch": "4 passes per replayed CUDA graph" if use_graph else "python, call by call",
                 "us_sharded_eager_python": round(us_sh_eager, 1)})
    for r in rows:
        if r["us_one_gpu"]:
            r["speedup_vs_one_gpu"] = round(r["us_one_gpu"] / r["us_sharded"], 3)
            r["efficiency"] = round(r["us_one_gpu"] / (world * r["us_sharded"]), 3)
    return {"world": world, "rows": rows,
            "note": "efficiency = t(one GPU, same tokens) / (N * t(N GPUs)); one token on N GPUs is bound by launch and collective latency, not by bytes"}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import moty_b200 as mb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        # a rank that fails must not leave the others waiting in a collective for NCCL's default ten minutes
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    mb.init([local])
    dev = torch.device("cuda", local)

    mats = make_inputs()
    W = [mb.Mat.i8(w, sc, device=local) for (w, sc, _) in mats]
    xs = [torch.from_numpy(x).to(dev) for (_, _, x) in mats]
    ys = [torch.empty((1, O), dtype=torch.float32, device=dev) for (O, _) in SHAPES]
    stream = torch.cuda.Stream(device=dev)
    sp = stream.cuda_stream
    total_bytes = sum(algo_bytes(*s) for s in SHAPES)

    # Every launch of this pass carries a few microseconds that are not streaming (launch, the per-CTA row quantizer,
    # the tail): for the 1-3 MB matrices that is ten times their HBM time.  The six products of a pass are independent,
    # so they go out as ONE launch (moty_cuda_mat_apply_multi_dev; --multi-max-mb caps the size of a matrix that joins,
    # --no-multi launches every matrix by itself).  Measured with the passes replayed as chained graphs: 53.5 us per
    # pass with six launches, 52.4 with the three small matrices in one, 51.0 with the 15360 x 3840 matrix in it as well,
    # 49.5 once that launch sized its units by row length, 47.95 with the 3840 x 15360 matrix (rows split in K) in it
    # too, and 46 with the dominant matrix as well.
    multi = [i for i in range(len(SHAPES)) if SHAPES[i][1] <= 16384 and
             SHAPES[i][0] * SHAPES[i][1] <= (args.multi_max_mb << 20)] if not args.no_multi else []
    if len(multi) < 2:
        multi = []
    # the launch the roofline is reported for: the one that holds the dominant matrix
    roof = multi if DOMINANT in multi else [DOMINANT]
    singles = [i for i in range(len(SHAPES)) if i not in multi]

    def launch(idxs):
        grp = [i for i in idxs if i in multi]
        if len(grp) > 1:
            mb.mat_apply_multi_dev([W[i] for i in grp], [ys[i].data_ptr() for i in grp], [xs[i].data_ptr() for i in grp], sp)
        else:
            grp = []
        for i in idxs:
            if i not in grp:
                mb.mat_apply_dev(W[i], ys[i].data_ptr(), xs[i].data_ptr(), 1, sp)
        return (1 if grp else 0) + len([i for i in idxs if i not in grp])

    def one_pass():
        return launch(list(range(len(SHAPES))))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            one_pass()
        barrier()
        sampler.start()
        # ---- device-resident passes ----
        K = args.steps
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # The K passes of the timed region are replayed from CUDA graphs of up to 32 whole passes each (a decode loop is
        # launch-bound otherwise), every launch chained to the next by programmatic dependent launch, so that a kernel's
        # prologue and first weight loads overlap the tail of the one before -- inside a pass and from one pass to the
        # next.  Nothing else sits in the timed region: an event record between two launches ends that overlap (measured:
        # 66 us per pass with the dominant launch bracketed by events, 52-55 us without).
        def capture(idxs, reps=1):
            if not idxs or reps < 1:
                return None
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for _ in range(reps):
                    launch(idxs)
            return g
        PER = min(K, 32)
        g_full = None if args.no_graph else capture(list(range(len(SHAPES))), PER)
        g_rest = None if args.no_graph else capture(list(range(len(SHAPES))), K % PER)
        # The timed region of K steps is repeated ROUNDS times (a region of K = 20 steps lasts about 1 ms: one sample of
        # that moved by 5 % between runs on different hosts); the median round is reported, each round bracketed by a
        # barrier and a device synchronisation on both sides.
        ROUNDS = 9
        round_ms = []
        for rnd in range(ROUNDS):
            barrier()
            e0.record(stream)
            if args.no_graph:
                for k in range(K):
                    one_pass()
            else:
                for k in range(K // PER):
                    g_full.replay()
                if g_rest is not None:
                    g_rest.replay()
            e1.record(stream)
            barrier()
            round_ms.append(e0.elapsed_time(e1))
        ms = statistics.median(round_ms)
        # The roofline's kernel: K further passes of the same sequence right after, now with the launch that holds the
        # dominant matrix issued directly between two events on its stream (what comes before and after it in the pass
        # replayed from two graphs), so that its own duration is measured in place, every launch of it streaming the
        # pass's 280 MB anew.  These passes are not part of `value`: the events cost the overlap described above.
        before = [i for i in range(0, min(roof)) if i not in roof]
        after = [i for i in range(len(SHAPES)) if i not in roof and i not in before]
        g_before = None if args.no_graph else capture(before)
        g_after = None if args.no_graph else capture(after)
        dom_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
        dom_all = []
        for rnd in range(3):
            barrier()
            for k in range(K):
                if args.no_graph:
                    launch(before)
                elif g_before is not None:
                    g_before.replay()
                dom_ev[k][0].record(stream)
                launch(roof)
                dom_ev[k][1].record(stream)
                if args.no_graph:
                    launch(after)
                elif g_after is not None:
                    g_after.replay()
            barrier()
            dom_all.append(statistics.mean(a.elapsed_time(b) for a, b in dom_ev))
        dom_ms = statistics.median(dom_all)

    # ---- end to end through the host-pointer entry, pinned host buffers ----
    hx = [mb.pinned_empty((1, I), np.float32) for (_, I) in SHAPES]
    hy = [mb.pinned_empty((1, O), np.float32) for (O, _) in SHAPES]
    for h, (_, _, x) in zip(hx, mats):
        h[...] = x
    for _ in range(3):
        for w, h_in, h_out in zip(W, hx, hy):
            mb.mat_apply(w, h_in, h_out)
    barrier()
    Ke = max(3, min(K, 200))
    t0 = time.perf_counter()
    for _ in range(Ke):
        for w, h_in, h_out in zip(W, hx, hy):
            mb.mat_apply(w, h_in, h_out)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop()

    # parity guard: the numbers above are only worth printing if the results are right.  Every matrix of the pass,
    # the dominant one included: all rows where the oracle takes milliseconds, a spread sample of rows otherwise
    # (an output row depends on its own weight row only, so a sampled row is checked exactly as in a full comparison)
    if rank == 0:
        from oracle import Oracle
        o = Oracle()
        prng = np.random.default_rng(99)
        for i in range(len(mats)):
            w, sc, x = mats[i]
            rows = np.arange(w.shape[0]) if w.shape[0] * w.shape[1] <= (8 << 20) else np.sort(prng.choice(w.shape[0], min(4096, w.shape[0]), replace=False))
            want = o.matmul_q_s(x, np.ascontiguousarray(w[rows]), sc[rows])
            got = ys[i].cpu().numpy()
            assert np.ascontiguousarray(got[:, rows]).tobytes() == want.tobytes(), f"GPU result differs from the oracle on matrix {i}"
            assert hy[i].tobytes() == got.tobytes(), f"host-pointer entry differs from the device entry on matrix {i}"

    if dist is not None:
        t = torch.tensor([ms, dom_ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, dom_ms, e2e_s = (float(v) for v in t.tolist())
    sharded = None
    if dist is not None and not args.no_extras:               # after the headline's numbers are final on every rank
        try:
            sharded = run_sharded(torch, dist, mb, dev, local, rank, world, K)
        except Exception as e:                                # an extra must not cost the headline line
            sharded = {"error": f"{type(e).__name__}: {e}"[:300]}
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    value = world * total_bytes * K / (ms * 1e-3) / 1e9
    e2e = world * total_bytes * Ke / e2e_s / 1e9
    peak, peak_kind = measured_peak()
    roof_bytes = sum(algo_bytes(*SHAPES[i]) for i in roof)
    isolated_ms = dom_ms
    whole_pass = len(roof) == len(SHAPES)
    if whole_pass:
        # the pass IS this kernel: its average launch duration over the timed region is the region's own events / K
        dom_ms = ms / K
    achieved = roof_bytes / (dom_ms * 1e-3) / 1e9
    if len(roof) > 1:
        roof_kernel = (f"q8_multi_kernel, {len(roof)} matrices of the pass in one launch (" +
                       ", ".join(f"{SHAPES[i][0]}x{SHAPES[i][1]}" for i in roof) + "), S=1")
        roof_profile = "q8_multi_sweep_pass.md"
    else:
        roof_kernel = "q8_stream_kernel<1,4,2,fused> 151936x1024 S=1"
        roof_profile = "q8_stream_gemv_151936x1024.md"
    roof_traffic = profile_traffic(roof_profile)
    cpu = None
    if world == 1 and not args.no_cpu:
        gbs, cores, kind, done, dt = cpu_arm(mats, 10 ** 9, 1, budget_s=12.0)
        cpu = {"value": round(gbs, 3), "unit": "GB/s", "cores": cores, "kind": kind,
               "sample": f"{done} passes of the same sweep with moty_matmul_q_s, {dt:.1f} s"}
    extras = None
    if world == 1 and not args.no_extras and len(SHAPES) == 6:
        extras = run_extras(torch, mb, dev, stream, W, local)
    if sharded is not None:
        extras = {"sharded": sharded}
    line = {"metric": METRIC, "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms / K, 6), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8xint8->int32", "data": "synthetic",
            "config": config_dict(world),
            "launch": ("direct" if args.no_graph else f"cuda_graph_replay, {min(K, 32)} passes per graph, launches chained by programmatic dependent launch") +
                      (f"; the {len(multi)} matrices of at most {args.multi_max_mb} MB in one launch" if len(multi) > 1 else ""),
            "timed_region": f"median of {ROUNDS} rounds of {K} steps",
            "pct_of_8TBs": round(100 * value / world / 8000.0, 2),
            "roofline": {"bound": "hbm", "kernel": roof_kernel, "achieved": round(achieved, 1),
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                         "traffic": roof_traffic,
                         "traffic_source": (f"committed ncu summary profiles/{roof_profile} (dram read + write bytes of one launch of this kernel), "
                                            "not measured in this run") if roof_traffic is not None else None,
                         "algorithmic_bytes": roof_bytes,
                         "avg_launch_us": round(dom_ms * 1e3, 3),
                         "isolated_launch_us": round(isolated_ms * 1e3, 3),
                         "timing": ((f"avg_launch_us: the timed region is {K} launches of this kernel and nothing else, CUDA events around "
                                     "them on the launch stream / their number; ") if whole_pass else
                                    (f"avg_launch_us: CUDA events around this kernel's launch in {K} further passes of the same sequence, "
                                     "right after the timed region; ")) +
                                   (f"isolated_launch_us: one launch between two events, in {K} further passes right after the timed region "
                                    "(an event between two launches ends their overlap: launch latency, first loads and tail are then exposed)")},
            "cpu_baseline": cpu,
            "e2e": {"value": round(e2e, 2), "unit": "GB/s", "steps": Ke,
                    "h2d_bytes_per_step": sum(4 * I for (_, I) in SHAPES), "d2h_bytes_per_step": sum(4 * O for (O, _) in SHAPES)},
            "gpu_launches": K * ((1 if len(multi) > 1 else len(multi)) + len(singles)), "clocks": clocks,
            "decode_tok_s": decode_summary(extras), "extras": extras}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_ep_case(args, name, S):
    """Expert-parallel MoE layer over the ranks of a torchrun launch (moty_b200/parallel.py): experts in
    contiguous ranges per rank, S tokens per rank, routing at home, all-to-all out and back, ordered combine.
    Prints the time per layer call (CUDA events, max over ranks) beside the same S * world tokens on one GPU."""
    import torch
    import torch.distributed as dist
    import moty_b200 as mb
    from moty_b200.parallel import ExpertParallelMoe
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    mb.init([local])
    E, K, I, D, f = MOE_SHAPES[name]
    fmt = mb.WF_I8 if f == "i8" else mb.WF_Q4R4
    rng = np.random.default_rng(5)
    ep = ExpertParallelMoe(E, K, I, D, efmt=fmt, device=local)
    one = mb.Moe(E, K, I, D, efmt=fmt, device=local) if rank == 0 else None
    for e in range(E):
        if fmt == mb.WF_I8:
            g = rng.integers(-127, 128, (I, D), dtype=np.int8); u = rng.integers(-127, 128, (I, D), dtype=np.int8)
            d = rng.integers(-127, 128, (D, I), dtype=np.int8)
            gs = rng.uniform(0.001, 0.02, I).astype(np.float32); us = rng.uniform(0.001, 0.02, I).astype(np.float32)
            ds = rng.uniform(0.001, 0.02, D).astype(np.float32)
        else:
            ng, nd = (I // 4) * (D // 32), (D // 4) * (I // 32)
            g = rng.integers(0, 256, ng * 64, dtype=np.uint8); u = rng.integers(0, 256, ng * 64, dtype=np.uint8)
            d = rng.integers(0, 256, nd * 64, dtype=np.uint8)
            gs = np.full(ng * 4, 0x1A00, np.uint16); us = np.full(ng * 4, 0x1A00, np.uint16); ds = np.full(nd * 4, 0x1A00, np.uint16)
        ep.upload_expert(e, g, gs, u, us, d, ds)
        if one is not None:
            one.upload_expert(e, g, gs, u, us, d, ds)
    x = torch.randn((S, D), device=dev); logits = torch.randn((S, E), device=dev)

    def timed(fn, n):
        for _ in range(3):
            fn()
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    us_ep = timed(lambda: ep.forward(x, logits, order=1), max(args.steps, 3))
    us_one = None
    if rank == 0:
        xa = torch.randn((S * world, D), device=dev); la = torch.randn((S * world, E), device=dev); oa = torch.empty_like(xa)
        st = mb.stream_handle(torch.cuda.current_stream())
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            one.apply_dev(oa.data_ptr(), xa.data_ptr(), S * world, la.data_ptr(), 1, 1, 0, 0, st)
        torch.cuda.synchronize(); e0.record()
        for _ in range(max(args.steps, 3)):
            one.apply_dev(oa.data_ptr(), xa.data_ptr(), S * world, la.data_ptr(), 1, 1, 0, 0, st)
        e1.record(); torch.cuda.synchronize()
        us_one = e0.elapsed_time(e1) * 1e3 / max(args.steps, 3)
    dist.barrier()
    if rank == 0:
        print(json.dumps({"case": args.case, "world": world, "tokens_per_rank": S, "us_per_layer_ep": round(us_ep, 1),
                          "us_per_layer_one_gpu_same_tokens": round(us_one, 1)}), flush=True)
    dist.destroy_process_group()


def run_case(args):
    """One matrix product, launched --warmup + --steps times on one stream (a small, self-ending
    workload for ncu captures of a single kernel)."""
    import torch
    import moty_b200 as mb
    parts = args.case.split(":")
    if parts[0] == "ep":                                       # ep:NAME:S -- run under torchrun: expert-parallel layer, S tokens per rank
        run_ep_case(args, parts[1], int(parts[2]))
        return
    mb.init([0])
    if args.fast_path >= 0:
        mb.lib().moty_cuda_set_moe_fast_path(args.fast_path)
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    if parts[0] == "moe":                                      # moe:NAME:S -- layer calls of a routed layer, two weight sets
        name, S = parts[1], int(parts[2])
        if len(parts) > 3 and parts[3] == "relaxed":       # moe:NAME:S:relaxed -- Q4R4 grouped products with the opt-in switch
            mb.lib().moty_cuda_set_q4r4_batch_relaxed(1)
        layers, per_expert = make_moe_layers(mb, name, 2, 0, rng)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            us = time_moe(torch, layers, name, S, dev, stream, reps=max(1, args.steps // 16), run=16)
        print(json.dumps({"case": args.case, "us_per_layer": round(us, 2)}), flush=True)
        return
    if parts[0] == "decode" and parts[1] in ("olmoe", "qwen3-30b-a3b"):
        # decode:olmoe[:NGEN] -- configs[2] shape: int8 attention matrices and experts, 16 layers, 16 heads
        # decode:qwen3-30b-a3b[:NGEN] -- configs[3] shape: Q4R4 attention matrices and experts, 48 layers, 32 query / 4 KV
        #   heads, 128 experts top-8 of width 768, top-k weights renormalised; the tied head stays int8 as in the reference
        #   (load_embed_q8).  Four weight sets are cycled over the layers in both.
        import time
        from moty_b200.decoder import DenseDecoder, DenseLayer
        name = parts[1]
        ngen = int(parts[2]) if len(parts) > 2 else 256
        if name == "olmoe":
            NL, D, H, KVH, hd, V, PROMPT, norm_topk = 16, 2048, 16, 16, 128, 50304, 512, 0
        else:
            NL, D, H, KVH, hd, V, PROMPT, norm_topk = 48, 2048, 32, 4, 128, 151936, 512, 1
        E, K, I, _, efmt = MOE_SHAPES[name]
        moes, per_expert = make_moe_layers(mb, name, 4, 0, rng)             # four expert sets, cycled over the layers
        for m in moes:
            m.set_router(mb.Mat.f32((rng.standard_normal((E, D)) * 0.02).astype(np.float32), device=0))
        one = lambda n: np.ones(n, np.float32)
        raw = lambda O, Kk: (rng.integers(-127, 128, (O, Kk), dtype=np.int8), rng.uniform(0.0002, 0.0006, O).astype(np.float32))
        def q4mat(O, Kk):                               # random Q4R4 codes, f16 scale 0.00293 (outputs of the size of the inputs)
            nblk, nb = (O + 3) // 4, Kk // 32
            return mb.Mat.q4r4(rng.integers(0, 256, nblk * nb * 64, dtype=np.uint8), np.full(nblk * nb * 4, 0x1A00, np.uint16), O, Kk, device=0)
        qw, kw = H * hd, KVH * hd
        sets = []
        for i in range(4):
            if efmt == "i8":
                q, k, v = raw(qw, D), raw(kw, D), raw(kw, D)
                qkv = mb.Mat.i8(np.concatenate([q[0], k[0], v[0]]), np.concatenate([q[1], k[1], v[1]]), device=0)
                sets.append((mb.Mat.i8(*q, device=0), mb.Mat.i8(*k, device=0), mb.Mat.i8(*v, device=0), mb.Mat.i8(*raw(D, qw), device=0), qkv))
                attn_bytes = 2 * D * qw + 2 * D * kw
            else:
                sets.append((q4mat(qw, D), q4mat(kw, D), q4mat(kw, D), q4mat(D, qw), q4mat(qw + 2 * kw, D)))
                attn_bytes = (2 * D * qw + 2 * D * kw) * 72 // 128
        layers = []
        for i in range(NL):
            q, k, v, o, qkv = sets[i % 4]
            layers.append(DenseLayer(q, k, v, o, None, None, None, one(D), one(D), one(hd), one(hd), qkv=qkv, moe=moes[i % 4], norm_topk=norm_topk))
        head = mb.Mat.i8(rng.integers(-127, 128, (V, D), dtype=np.int8), rng.uniform(0.005, 0.015, V).astype(np.float32), device=0)
        dec = DenseDecoder(layers, head, one(D), H, KVH, hd, PROMPT + ngen + 8, max_S=PROMPT)
        prompt = np.random.default_rng(1).integers(0, V, PROMPT).astype(np.int32)
        dec.step(prompt, 0); dec.step([1], PROMPT)
        torch.cuda.synchronize(); t0 = time.perf_counter()
        tok = dec.step(prompt, 0)
        torch.cuda.synchronize(); t1 = time.perf_counter()
        toks = [tok]
        for i in range(ngen):
            toks.append(dec.step([toks[-1]], PROMPT + i))
        torch.cuda.synchronize(); t2 = time.perf_counter()
        tg = dec.greedy_graph(tok, PROMPT, ngen)
        torch.cuda.synchronize(); t3 = time.perf_counter()
        tg = dec.greedy_graph(tok, PROMPT, ngen)
        torch.cuda.synchronize(); t4 = time.perf_counter()
        wbytes = NL * (K * per_expert + attn_bytes + 4 * E * D) + head.nbytes()
        print(json.dumps({"case": args.case, "prefill_tok_s": round(PROMPT / (t1 - t0), 1), "decode_tok_s": round(ngen / (t2 - t1), 1),
                          "ms_per_token": round((t2 - t1) / ngen * 1e3, 3), "weight_MB_per_token": round(wbytes / 1e6, 1),
                          "graph_decode_tok_s": round(ngen / (t4 - t3), 1), "graph_ms_per_token": round((t4 - t3) / ngen * 1e3, 3),
                          "graph_GBs": round(wbytes * ngen / (t4 - t3) / 1e9, 1), "graph_equals_direct": tg == toks[1:]}), flush=True)
        dec.close()
        return
    if parts[0] == "decode" and parts[1] == "gemma":    # decode:gemma[:NGEN[:PROMPT[:NL]]] -- configs[4] shape, synthetic int8 weights
        import time
        from moty_b200.decoder import GemmaDecoder, GemmaLayer
        ngen = int(parts[2]) if len(parts) > 2 else 256
        PROMPT = int(parts[3]) if len(parts) > 3 else 4096
        NL = int(parts[4]) if len(parts) > 4 else 48
        D, H, KV, hd, I, V, WINDOW = 3840, 16, 8, 256, 15360, 262144, 1024
        def raw(O, Kk, lo=0.0002, hi=0.0006):
            q = np.frombuffer(rng.bytes(O * Kk), np.int8).reshape(O, Kk)
            return np.maximum(q, -127), rng.uniform(lo, hi, O).astype(np.float32)
        mk = lambda O, Kk: mb.Mat.i8(*raw(O, Kk), device=0)
        one = lambda n: np.ones(n, np.float32)
        layers = []
        for i in range(NL):
            q, k, v = raw(H * hd, D), raw(KV * hd, D), raw(KV * hd, D)
            qkv = mb.Mat.i8(np.concatenate([q[0], k[0], v[0]]), np.concatenate([q[1], k[1], v[1]]), device=0)
            sliding = (i + 1) % 6 != 0                                  # 5 of every 6 layers slide, the sixth is global
            layers.append(GemmaLayer(mb.Mat.i8(*q, device=0), mb.Mat.i8(*k, device=0), mb.Mat.i8(*v, device=0), mk(D, H * hd),
                                     mk(I, D), mk(I, D), mk(D, I), one(D), one(D), one(D), one(D), one(hd), one(hd), one(hd),
                                     n_kv_heads=KV, head_dim=hd, theta=1e4 if sliding else 1e6, window=WINDOW if sliding else 0, qkv=qkv))
        head = mb.Mat.i8(*raw(V, D, 0.0001, 0.0003), device=0)
        dec = GemmaDecoder(layers, head, one(D), H, PROMPT + ngen + 8, max_S=512)
        prompt = np.random.default_rng(1).integers(0, V, PROMPT).astype(np.int32)
        dec.prefill(prompt[:min(PROMPT, 512)], 0); dec.step([1], min(PROMPT, 512))      # warm-up (allocations, attributes)
        torch.cuda.synchronize(); t0 = time.perf_counter()
        tok = dec.prefill(prompt, 0, block=512)
        torch.cuda.synchronize(); t1 = time.perf_counter()
        toks = [tok]
        for i in range(ngen):
            toks.append(dec.step([toks[-1]], PROMPT + i))
        torch.cuda.synchronize(); t2 = time.perf_counter()
        tg = dec.greedy_graph(tok, PROMPT, ngen)
        torch.cuda.synchronize(); t3 = time.perf_counter()
        tg = dec.greedy_graph(tok, PROMPT, ngen)
        torch.cuda.synchronize(); t4 = time.perf_counter()
        wbytes = sum(m.nbytes() for l in layers for m in (l.qkv, l.o, l.gate, l.up, l.down)) + head.nbytes()
        print(json.dumps({"case": args.case, "layers": NL, "prompt": PROMPT, "prefill_tok_s": round(PROMPT / (t1 - t0), 1),
                          "prefill_s": round(t1 - t0, 3), "decode_tok_s": round(ngen / (t2 - t1), 1),
                          "ms_per_token": round((t2 - t1) / ngen * 1e3, 3), "weight_MB_per_token": round(wbytes / 1e6, 1),
                          "graph_decode_tok_s": round(ngen / (t4 - t3), 1), "graph_ms_per_token": round((t4 - t3) / ngen * 1e3, 3),
                          "graph_GBs": round(wbytes * ngen / (t4 - t3) / 1e9, 1), "graph_equals_direct": tg == toks[1:]}), flush=True)
        dec.close()
        return
    if parts[0] == "decode":                            # decode:qwen3-0.6b[:NGEN] -- configs[0] shape, synthetic int8 weights
        fold = {"fold": True, "nofold": False}.get(parts[3]) if len(parts) > 3 else None      # decode:qwen3-0.6b:NGEN[:fold|nofold]
        res = run_decode_qwen(torch, mb, rng, int(parts[2]) if len(parts) > 2 else 128, 0, fold)
        print(json.dumps({"case": args.case, **res}), flush=True)
        return
    if parts[0] == "attn":                              # attn:S:POS:H:KV:hd[:kv8][:posdev] -- S tokens at position POS of one layer's cache
        S, POS, H, KV, hd = (int(v) for v in parts[1:6])
        kv8 = "kv8" in parts[6:]
        posdev = "posdev" in parts[6:]                  # position read from the device: with S = 1 the one-launch decode core
        a = mb.Attn(H, KV, hd, POS + S, qn=np.ones(hd, np.float32), kn=np.ones(hd, np.float32), kv8=kv8)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            q0 = torch.randn((S, H * hd), device=dev); k0 = torch.randn((S, KV * hd), device=dev)
            q = q0.clone(); k = k0.clone(); v = torch.randn((S, KV * hd), device=dev); ctx = torch.empty((S, H * hd), device=dev)
            run = lambda: a.core_dev(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), S, POS, stream=stream.cuda_stream)
            if posdev:
                pd = torch.full((1,), POS, device=dev, dtype=torch.int32)
                run = lambda: a.core_posdev(ctx.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), S, pd.data_ptr(), POS,
                                            stream=stream.cuda_stream)
            for _ in range(max(args.warmup, 1)):
                run()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                run()
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        kvb = 2.0 * KV * (POS + S) * hd * (1 if kv8 else 4)           # cache bytes a decode step reads
        print(json.dumps({"case": args.case, "us": round(us, 2), "kv_GBs": round(kvb / us / 1e3, 1)}), flush=True)
        return
    if parts[0] == "ffn":                               # ffn:S:D:I -- one dense int8 SiLU FFN block (gate/up [I][D], down [D][I])
        S, D, I = int(parts[1]), int(parts[2]), int(parts[3])
        mk = lambda O, K: mb.Mat.i8(rng.integers(-127, 128, (O, K), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32), device=0)
        G, U, Dn = mk(I, D), mk(I, D), mk(D, I)
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            x = torch.randn((S, D), device=dev); y = torch.empty((S, D), device=dev)
            for _ in range(max(args.warmup, 1)):
                mb.dense_ffn_dev(G, U, Dn, y.data_ptr(), x.data_ptr(), S, stream=stream.cuda_stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                mb.dense_ffn_dev(G, U, Dn, y.data_ptr(), x.data_ptr(), S, stream=stream.cuda_stream)
            e1.record(stream)
            torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / args.steps
        print(json.dumps({"case": args.case, "us_per_block": round(us, 2), "GBs": round(3.0 * I * D / us / 1e3, 1)}), flush=True)
        return
    fmt, S, O, I = parts
    S, O, I = int(S), int(O), int(I)
    if fmt in ("q4r4x", "q8r4x"):                       # the batch kernel with one formula for every token (opt-in switch)
        mb.lib().moty_cuda_set_q4r4_batch_relaxed(1)
        fmt = fmt[:-1]
    if fmt == "q8_0":
        w = mb.Mat.i8(rng.integers(-127, 128, (O, I), dtype=np.int8), rng.uniform(0.001, 0.02, O).astype(np.float32), device=0)
        nbytes = algo_bytes(O, I, S)
    elif fmt == "i4g":
        w = mb.Mat.i4g(rng.integers(0, 256, (O, I // 2), dtype=np.uint8), rng.uniform(0.001, 0.02, (O, I // 32)).astype(np.float32), O, I, device=0)
        nbytes = O * I // 2 + 4 * O * (I // 32) + 4 * S * I + 4 * S * O
    elif fmt == "q8r4":
        nblk, nb = (O + 3) // 4, I // 32
        w = mb.Mat.q8r4(rng.integers(-127, 128, nblk * nb * 128, dtype=np.int8), np.full(nblk * nb * 4, 0x1A00, np.uint16), O, I, device=0)
        nbytes = nblk * nb * 136 + 4 * S * I + 4 * S * O
    else:
        nblk, nb = (O + 3) // 4, I // 32
        w = mb.Mat.q4r4(rng.integers(0, 256, nblk * nb * 64, dtype=np.uint8), np.full(nblk * nb * 4, 0x1A00, np.uint16), O, I, device=0)
        nbytes = q4r4_bytes(O, I, S)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        x = torch.randn((S, I), device=dev); y = torch.empty((S, O), device=dev)
        for _ in range(max(args.warmup, 1)):
            mb.mat_apply_dev(w, y.data_ptr(), x.data_ptr(), S, stream.cuda_stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            mb.mat_apply_dev(w, y.data_ptr(), x.data_ptr(), S, stream.cuda_stream)
        e1.record(stream)
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / args.steps
    print(json.dumps({"case": args.case, "us": round(us, 2), "GBs": round(nbytes / us / 1e3, 1),
                      "TOPS": round(2.0 * S * O * I / us / 1e6, 2), "steps": args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--shapes", default="", help="comma-separated indices into the sweep (profiling aid); default all six")
    ap.add_argument("--multi-max-mb", type=int, default=256, help="largest matrix (MB) that joins the several-products-in-one-launch call")
    ap.add_argument("--no-multi", action="store_true", help="launch the small matrices one by one instead of in one launch")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling aid)")
    ap.add_argument("--no-graph", action="store_true", help="launch every GEMV directly instead of replaying CUDA graphs")
    ap.add_argument("--fast-path", type=int, default=-1, help="profiling aid for --case: 0/1/2 passed to moty_cuda_set_moe_fast_path "
                                                            "(0 = step-by-step FFN and general MoE path, 1 = one-launch decode kernels)")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-shape S=16/512 and Q4R4 rows")
    ap.add_argument("--case", default="", help="profiling aid: FMT:S:O:I (FMT q8_0, q4r4 or q8r4) times only that product, "
                                                "--steps launches after --warmup; moe:NAME:S (NAME olmoe or qwen3-30b-a3b) "
                                                "times calls of one routed layer; decode:qwen3-0.6b[:NGEN] a 64-token prompt and NGEN greedy steps of the configs[0]-shaped dense decoder, decode:olmoe[:NGEN] a 512-token prompt and NGEN steps of the configs[2]-shaped MoE decoder; decode:gemma[:NGEN[:PROMPT[:NL]]] a PROMPT-token (4096) blocked prefill and NGEN (256) steps of the configs[4]-shaped dense decoder with NL (48) layers; ffn:S:D:I one dense int8 SiLU FFN block; attn:S:POS:H:KV:hd[:kv8][:posdev] the attention core with S tokens at position POS (posdev: position read from the device, the one-launch decode core); ep:NAME:S under torchrun times the "
                                                "expert-parallel layer with S tokens per rank; prints one row and exits")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    if args.shapes:
        global SHAPES, DOMINANT, WORKLOAD
        keep = [int(v) for v in args.shapes.split(",")]
        dom = SHAPES[DOMINANT]
        SHAPES = [SHAPES[i] for i in keep]
        DOMINANT = SHAPES.index(dom) if dom in SHAPES else 0
        WORKLOAD += f" (subset {keep})"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
