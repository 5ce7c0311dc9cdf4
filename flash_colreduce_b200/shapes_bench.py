"""Latency / peak-memory table over the reference's 20 benchmark shapes.

    python -m flash_colreduce_b200.shapes_bench [--naive] [--json out.json]

Counterpart of the reference's ``benchmarks/run.py`` (shape list :11-56,
calibrated wall-clock latency :59-83, peak memory :86-92, h=32, d=128, fp16,
reduction "sum"): the same 20 configurations, measured the same way, so that
the rows line up with ``benchmarks/results/*.log``.  ``--naive`` also times the
materialising definition where its (B,H,M,N) matrix fits, chunked over batch
like the reference's ``chunked_run`` (:95-131).
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from . import flash_colreduce, naive_colreduce, valid_scores

SHAPES = (
    [dict(b=b, h=32, m=1024, n=1024, d=128, is_causal=False) for b in (1, 4, 16, 64, 256)]
    + [dict(b=1, h=32, m=n, n=n, d=128, is_causal=False) for n in (1024, 2048, 4096, 8192, 16384)]
    + [dict(b=b, h=32, m=64, n=16384, d=128, is_causal=True) for b in (1, 4, 16, 64, 256)]
    + [dict(b=1, h=32, m=512, n=n, d=128, is_causal=True) for n in (16384, 32768, 65536, 131072, 262144)]
)


def _now() -> float:
    torch.cuda.synchronize()
    return time.perf_counter()


@torch.inference_mode()
def measure_latency(fn, min_iters: int = 10) -> float:
    """One call, a 10-call calibration, then as many warm-up and timed calls as fit in about a second."""
    torch.cuda.empty_cache()
    fn()
    start = _now()
    for _ in range(min_iters):
        fn()
    iters = max(int(min_iters / max(_now() - start, 1e-9)), min_iters)
    iters = min(iters, 2000)
    for _ in range(iters):
        fn()
    start = _now()
    for _ in range(iters):
        fn()
    return (_now() - start) / iters


@torch.inference_mode()
def measure_memory(fn) -> int:
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    fn()
    torch.cuda.synchronize()
    return torch.cuda.max_memory_allocated()


def _naive_chunked(q, k, is_causal, budget_bytes=8 << 30):
    b, h, m, d = q.shape
    n = k.shape[2]
    per_batch = h * m * n * 2 * 4  # a few fp16 copies of the score matrix
    step = max(1, min(b, budget_bytes // max(per_batch, 1)))
    out = torch.empty((b, h, n), dtype=q.dtype, device=q.device)
    for lo in range(0, b, step):
        out[lo:lo + step] = naive_colreduce(q[lo:lo + step], k[lo:lo + step], "sum", is_causal)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--naive", action="store_true", help="also time the materialising definition on the GPU")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    print(f"GPU: {torch.cuda.get_device_name(dev)}")
    rows = []
    head = f"{'config':46s} {'flash ms':>9s} {'flash MB':>9s} {'Gscores/s':>10s} {'TFLOP/s':>8s}"
    if args.naive:
        head += f" {'naive ms':>9s} {'speedup':>8s}"
    print(head)
    for cfg in SHAPES:
        b, h, m, n, d, causal = cfg["b"], cfg["h"], cfg["m"], cfg["n"], cfg["d"], cfg["is_causal"]
        q = torch.randn(b, h, m, d, device=dev, dtype=torch.float16)
        k = torch.randn(b, h, n, d, device=dev, dtype=torch.float16)
        fn = lambda: flash_colreduce(q, k, "sum", is_causal=causal)
        lat = measure_latency(fn)
        mem = measure_memory(fn)
        scores = valid_scores(b, h, m, n, causal)
        row = dict(cfg, flash_ms=lat * 1e3, flash_mb=mem / 2**20, gscores_per_s=scores / lat / 1e9,
                   tflops=4 * d * scores / lat / 1e12)
        line = (f"b={b:<3d} h={h} m={m:<6d} n={n:<6d} d={d} causal={str(causal):5s} "
                f"{row['flash_ms']:9.3f} {row['flash_mb']:9.1f} {row['gscores_per_s']:10.1f} {row['tflops']:8.1f}")
        if args.naive and b * h * m * n <= 2**34:
            nlat = measure_latency(lambda: _naive_chunked(q, k, causal), min_iters=3)
            row.update(naive_ms=nlat * 1e3, speedup=nlat / lat)
            line += f" {row['naive_ms']:9.3f} {row['speedup']:8.2f}"
        print(line, flush=True)
        rows.append(row)
        del q, k
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
