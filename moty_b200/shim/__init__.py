"""Reference-side shim: the C file a maintainer adds to the reference (hw_cuda.c), a wrapper translation
unit that builds the reference's own `qwen` engine with it (qwen_cuda.c), the recipe (Makefile) and a
writer of synthetic snapshots (make_snapshot.py).  `engine_binary()` finds the built engine; `run_engine()`
runs it in REF= validation mode on the CPU (the reference as it is) or with the matmuls on a GPU."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")


def build(ref_src: str | None = None) -> None:
    """Compile the engine + shim where the reference checkout is present (a no-op message otherwise)."""
    ref_src = ref_src or os.environ.get("MOTY_REF_SRC", "")
    subprocess.check_call(["make", "-s", "-C", HERE, "all"] + ([f"REF={ref_src}"] if ref_src else []))


def _cpu_has(flag: str) -> bool:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return flag in line.split()
    except OSError:
        pass
    return False


def engine_binary() -> str | None:
    """The tier this CPU can run: the build host's native tier when it needs no AVX512-VNNI or the CPU has it, else AVX2."""
    native, v3 = os.path.join(BUILD, "qwen_cuda_native"), os.path.join(BUILD, "qwen_cuda_v3")
    need = os.path.join(BUILD, "native_needs_avx512vnni")
    if os.path.exists(native):
        needs = os.path.exists(need) and open(need).read().strip() not in ("", "0")
        if not needs or (_cpu_has("avx512_vnni") and _cpu_has("avx512bw")):
            return native
    return v3 if os.path.exists(v3) else None


def run_engine(snap: str, cuda, trace: str | None = None, qbits: int = 8, threads: int | None = None,
               gpu: int = 0, extra_env: dict | None = None, timeout: float = 1200) -> subprocess.CompletedProcess:
    """SNAP=<snap> QBITS=<qbits> REF=<snap>/ref.json [MOTY_CUDA=1] qwen_cuda, output captured."""
    exe = engine_binary()
    if exe is None:
        raise RuntimeError("the shimmed engine is not built (make -C moty_b200/shim needs the reference checkout)")
    env = dict(os.environ, SNAP=snap, QBITS=str(qbits), REF=os.path.join(snap, "ref.json"), MOTY_NO_OMP_TUNE="1",
               MOTY_CUDA=str(int(cuda)), MOTY_GPU=str(gpu))       # 0 = CPU, 1 = mat_apply hook, 2 = whole step on the GPU
    if trace:
        env["MOTY_SHIM_TRACE"] = trace
    if threads:
        env["THREADS"] = str(threads)
    env.update(extra_env or {})
    return subprocess.run([exe], env=env, capture_output=True, text=True, timeout=timeout)
