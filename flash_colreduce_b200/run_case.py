"""Runs one synthetic case of the operator on the current GPU and prints its timing.

    python -m flash_colreduce_b200.run_case --heads 64 --m 8192 --n 8192 --d 128 --causal --reduction sum --iters 2

Handy for a quick check of an installation and as the small, self-ending
workload to put under a profiler (inputs larger than the L2, a few launches).
"""
from __future__ import annotations

import argparse

import torch

from . import flash_colreduce, valid_scores
from . import _native as nat


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--m", type=int, default=16384)
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--reduction", default="sum", choices=["sum", "mean", "max"])
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--bf16", action="store_true")
    ap.add_argument("--iters", type=int, default=2)
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if args.bf16 else torch.float16
    gen = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(args.batch, args.heads, args.m, args.d, generator=gen, device=dev, dtype=torch.float32).to(dtype)
    k = torch.randn(args.batch, args.heads, args.n, args.d, generator=gen, device=dev, dtype=torch.float32).to(dtype)
    nat.lib.fcr_trace_enable(1)
    for _ in range(max(args.iters, 1)):
        out = flash_colreduce(q, k, args.reduction, is_causal=args.causal)
    torch.cuda.synchronize()
    rows_ms, cols_ms = nat.trace_times()[-1]
    nat.lib.fcr_trace_enable(0)
    scores = valid_scores(args.batch, args.heads, args.m, args.n, args.causal)
    ms = rows_ms + cols_ms
    print(f"B={args.batch} H={args.heads} M={args.m} N={args.n} D={args.d} {args.reduction} causal={args.causal} {dtype}: "
          f"rows pass {rows_ms:.3f} ms, columns pass {cols_ms:.3f} ms, {scores / ms / 1e6:.1f} Gscores/s, "
          f"{4 * args.d * scores / ms / 1e9:.1f} TFLOP/s, checksum {float(out.float().sum()):.6g}")


if __name__ == "__main__":
    main()
