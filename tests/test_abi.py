"""CPU: the C-ABI library loads, exports exactly what include/moty_cuda.h declares,
and fails loudly (no CPU fallback) when there is no GPU."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared():
    text = open(os.path.join(ROOT, "include", "moty_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moty_cuda_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    import moty_b200 as mb
    from moty_b200.build import build
    build()
    lib = mb.lib()
    names = declared()
    assert len(names) >= 40
    for n in names:
        assert hasattr(lib, n), f"{n} declared in moty_cuda.h but not exported"
    out = subprocess.run(["nm", "-D", "--defined-only", mb.LIB_PATH], capture_output=True, text=True).stdout
    exported = sorted(set(re.findall(r" T (moty_cuda_[a-z0-9_]+)", out)))
    assert exported == names, "exports and declarations differ"


def test_no_cpu_fallback_without_gpu():
    """Without a CUDA device every compute entry must return an error."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import moty_b200 as mb
    with pytest.raises(mb.MotyCudaError):
        mb.init([0])
    with pytest.raises(mb.MotyCudaError):
        mb.qrow_i8(np.ones((1, 32), np.float32))
    with pytest.raises(mb.MotyCudaError):
        mb.Mat.i8(np.ones((4, 16), np.int8), np.ones(4, np.float32))


def test_product_does_not_touch_the_oracle():
    """Nothing under moty_b200/ may import, link or open the CPU checkers."""
    pkg = os.path.join(ROOT, "moty_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
