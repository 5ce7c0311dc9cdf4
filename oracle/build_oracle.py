"""Compiles the C restatement ``colreduce_ref.c`` into ``oracle/_build/``.

TEST INFRASTRUCTURE ONLY.  Usage: ``python oracle/build_oracle.py``.
The reference itself is pure Python (no C/C++ sources to compile), so there is
no ``oracle/_ref`` build of it; the Python reference is instead executed in the
build container to produce ``tests/golden/``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "colreduce_ref.c")
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "libcolreduce_ref.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", LIB, SRC, "-lm"]
    subprocess.run(cmd, check=True)
    return LIB


def load() -> ctypes.CDLL:
    lib = ctypes.CDLL(build())
    lib.colreduce_ref.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                  ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_double]
    lib.colreduce_ref.restype = ctypes.c_int
    return lib


def colreduce_ref(q, k, reduction: str, is_causal: bool, scale: float):
    """numpy front end: q (B,H,M,D), k (B,H,N,D) float32 arrays -> (B,H,N) float64."""
    import numpy as np

    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    b, h, m, d = q.shape
    n = k.shape[2]
    out = np.zeros((b, h, n), dtype=np.float64)
    rc = load().colreduce_ref(q.ctypes.data, k.ctypes.data, out.ctypes.data, b * h, m, n, d,
                              {"sum": 0, "mean": 1, "max": 2}[reduction], 1 if is_causal else 0, float(scale))
    if rc != 0:
        raise RuntimeError("colreduce_ref rejected its arguments")
    return out


if __name__ == "__main__":
    print(build(force=True))
