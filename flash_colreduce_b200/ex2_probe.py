"""The benchmark's measurement of the exponential unit (``libfcr_ex2_probe.so``).

``ex2_rate()`` returns how many ``ex2.approx.ftz.f32`` the current GPU sustains
per second: the transcendental bound of the operator's roofline (one
exponential per attention score).  A helper of ``bench.py``; the operator does
not use it.
"""
from __future__ import annotations

import ctypes as C
import os

from .build import PROBE_PATH


def ex2_rate(repeats: int = 3) -> float:
    if not os.path.exists(PROBE_PATH):
        raise ImportError(f"{PROBE_PATH} is missing: build it with `python flash_colreduce_b200/build.py`")
    lib = C.CDLL(PROBE_PATH)
    lib.fcr_probe_ex2_rate.argtypes = [C.c_int32]
    lib.fcr_probe_ex2_rate.restype = C.c_double
    return float(lib.fcr_probe_ex2_rate(int(repeats)))
