"""Builds the sm_100a shared library of this package in-tree with nvcc.

Run as ``python flash_colreduce_b200/build.py`` (a script, so that it works before the
library exists).  nvcc cross-compiles, so no
GPU is needed.  The library lands next to this file in ``_lib/`` and is what
``flash_colreduce_b200._native`` loads; there is no JIT step and no fallback.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "_lib")
LIB_NAME = "libflash_colreduce_b200.so"
LIB_PATH = os.path.join(LIB_DIR, LIB_NAME)

SOURCES = ["colreduce_sm100.cu"]
# the benchmark's measurement helper, a library of its own (not part of the operator)
PROBE_NAME = "libfcr_ex2_probe.so"
PROBE_PATH = os.path.join(LIB_DIR, PROBE_NAME)
PROBE_SOURCES = ["ex2_probe.cu"]


def _dependencies() -> list:
    """Every file the library is compiled from: all of csrc/ and the public headers."""
    import glob

    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cuh")) +
                  glob.glob(os.path.join(CSRC, "*.h")) +
                  glob.glob(os.path.join(PKG_DIR, "..", "include", "*.h")))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-ldl",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH")


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(PROBE_PATH):
        return True
    built = min(os.path.getmtime(LIB_PATH), os.path.getmtime(PROBE_PATH))
    return any(os.path.getmtime(d) > built for d in _dependencies())


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if it is missing or older than its sources."""
    if not force and not is_stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    for target, sources in ((LIB_PATH, SOURCES), (PROBE_PATH, PROBE_SOURCES)):
        cmd = [_nvcc(), *NVCC_FLAGS]
        if target == LIB_PATH:
            cmd += os.environ.get("FCR_NVCC_EXTRA", "").split()  # tuning builds, e.g. -DFCR_POLY=3
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", target] + [os.path.join(CSRC, s) for s in sources]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed building " + os.path.basename(target))
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
