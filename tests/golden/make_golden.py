"""Generates ``naive_golden.npz``: outputs of the REFERENCE's own ``naive_colreduce``.

Run in the build container, where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/flash-colreduce

The reference is imported unmodified from that path and executed on the CPU
in fp32 on fp16-rounded inputs (the same bits the GPU kernels receive).  The
reference has no golden vectors of its own; these pin the oracle and the
kernels to it.  The file holds the fp16 inputs and the fp32 outputs, so that
nothing depends on a random-number generator staying stable.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, B, H, M, N, D, seed, scale)
INPUT_SETS = [
    ("c1", 2, 4, 256, 256, 64, 0, None),           # the reference's CPU-runnable benchmark configuration
    ("sq128_d16", 1, 1, 128, 128, 16, 1, None),    # the reference test matrix, tests/test_correctness.py:8-13
    ("sq131_d72", 1, 1, 131, 131, 72, 2, None),
    ("dec128_d72", 1, 1, 128, 1024, 72, 3, None),
    ("dec131_d16", 1, 1, 131, 1027, 16, 4, None),
    ("dec131_d32_h3", 1, 3, 131, 1027, 32, 5, None),
    ("tall300_d48", 1, 2, 300, 100, 48, 6, None),  # M > N: mean divisor quirk of naive.py:31-33
    ("scaled_d32", 2, 1, 140, 260, 32, 7, 0.3),    # user scale
]
REDUCTIONS = ("sum", "mean", "max")


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/flash-colreduce")
    ref_root = sys.argv[1]
    sys.path.insert(0, ref_root)
    from flash_colreduce.naive import naive_colreduce  # the reference, unmodified

    torch.set_num_threads(1)
    store = {}
    for name, b, h, m, n, d, seed, scale in INPUT_SETS:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, h, m, d, generator=g, dtype=torch.float32).half()
        k = torch.randn(b, h, n, d, generator=g, dtype=torch.float32).half()
        store[f"in__{name}__q"] = q.numpy()
        store[f"in__{name}__k"] = k.numpy()
        store[f"in__{name}__scale"] = np.array(-1.0 if scale is None else scale, dtype=np.float64)
        reds = ("sum",) if name == "c1" else REDUCTIONS
        causals = (False,) if name == "c1" else (False, True)
        for red in reds:
            for causal in causals:
                out = naive_colreduce(q.float(), k.float(), red, is_causal=causal, scale=scale)
                assert out.dtype == torch.float32 and out.shape == (b, h, n)
                store[f"out__{name}__{red}__{int(causal)}"] = out.numpy()
    path = os.path.join(HERE, "naive_golden.npz")
    np.savez_compressed(path, **store)
    print(path, os.path.getsize(path), "bytes,", sum(1 for key in store if key.startswith("out__")), "outputs")


if __name__ == "__main__":
    main()
