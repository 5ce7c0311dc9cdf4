"""Latency / peak-memory table over the reference's 20 benchmark shapes, side by side.

    python -m flash_colreduce_b200.shapes_bench [--reference-path DIR] [--naive] [--configs] [--cpu]
                                                [--slice-m] [--seconds S] [--json F] [--md F]

Counterpart of the reference's ``benchmarks/run.py`` (shape list :11-56,
calibrated wall-clock latency :59-83, peak memory :86-92, chunked calls
:95-131, side-by-side columns :134-179; h=32, d=128, fp16, reduction "sum"):
the same 20 rows in the same order, measured the same way, so that the table
lines up with ``benchmarks/results/*.log``.  Every row times

* this library's ``flash_colreduce``;
* with ``--reference-path DIR``: the unmodified reference package imported from
  ``DIR`` (its Triton kernel, compiled on this GPU by Triton's own JIT) on the
  same tensors -- a baseline beside the product, never part of it;
* with ``--naive``: the materialising definition on the GPU, chunked over batch
  and query rows when its (B,H,M,N) matrix does not fit, like ``chunked_run``.

``--configs`` appends the configurations the throughput metric is quoted on
(the 256-square CPU-sized case, square 512 x 3 reductions, causal decode 128 x 4096 x 3 reductions, the
8192-square VLM pruning shape, an 8-head shard of the 131072-square long
context); ``--cpu`` adds the definition on the host cores (fp32, all threads) for them.  ``--slice-m`` also times this library on query-row slices of one
larger tensor (non-contiguous views, the call pattern ``chunked_run`` produces).
"""
from __future__ import annotations

import argparse
import importlib
import json
import sys
import time

import torch

from . import flash_colreduce, naive_colreduce, valid_scores

SHAPES = (
    [dict(b=b, h=32, m=1024, n=1024, d=128, is_causal=False) for b in (1, 4, 16, 64, 256)]
    + [dict(b=1, h=32, m=n, n=n, d=128, is_causal=False) for n in (1024, 2048, 4096, 8192, 16384)]
    + [dict(b=b, h=32, m=64, n=16384, d=128, is_causal=True) for b in (1, 4, 16, 64, 256)]
    + [dict(b=1, h=32, m=512, n=n, d=128, is_causal=True) for n in (16384, 32768, 65536, 131072, 262144)]
)

METRIC_CONFIGS = (
    [dict(b=2, h=4, m=256, n=256, d=64, is_causal=False, reduction="sum", tag="c1")]
    + [dict(b=8, h=16, m=512, n=512, d=64, is_causal=False, reduction=r, tag="c2") for r in ("sum", "mean", "max")]
    + [dict(b=1, h=32, m=128, n=4096, d=128, is_causal=True, reduction=r, tag="c3") for r in ("sum", "mean", "max")]
    + [dict(b=4, h=32, m=8192, n=8192, d=128, is_causal=True, reduction="mean", tag="c4")]
    + [dict(b=1, h=8, m=131072, n=131072, d=128, is_causal=True, reduction="sum", tag="c5 shard (8 of 64 heads)")]
)


def _now() -> float:
    torch.cuda.synchronize()
    return time.perf_counter()


@torch.inference_mode()
def measure_latency(fn, min_iters: int = 10, seconds: float = 1.0) -> float:
    """One call, a 10-call calibration, then as many warm-up and timed calls as fit in ``seconds``."""
    torch.cuda.empty_cache()
    fn()
    start = _now()
    for _ in range(min_iters):
        fn()
    iters = max(int(seconds * min_iters / max(_now() - start, 1e-9)), min_iters)
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


_CHUNKS: dict = {}


def chunked_call(op, q, k, reduction, is_causal):
    """Calls ``op`` on batch / query-row slices small enough to fit, halving the slice on
    out-of-memory, and adds the pieces up; a size that worked is remembered per shape."""
    b, _, m, _ = q.shape
    n = k.shape[2]
    key = (id(op), tuple(q.shape), n, is_causal)
    cb, cm = _CHUNKS.get(key, (b, m))
    while True:
        try:
            out = torch.zeros((b, q.shape[1], n), device=q.device, dtype=q.dtype)
            for bl in range(0, b, cb):
                for ml in range(0, m, cm):
                    out[bl:bl + cb] += op(q[bl:bl + cb, :, ml:ml + cm], k[bl:bl + cb], reduction=reduction,
                                          is_causal=is_causal)
            _CHUNKS[key] = (cb, cm)
            return out
        except torch.OutOfMemoryError:
            if cb > 1:
                cb //= 2
            elif cm > 1:
                cm //= 2
            else:
                raise
            torch.cuda.empty_cache()


def _load_reference(path: str):
    """The reference package, imported from ``path`` (its operator and its materialising definition)."""
    sys.path.insert(0, path)
    try:
        mod = importlib.import_module("flash_colreduce")
    finally:
        sys.path.remove(path)
    return mod


def _label(cfg) -> str:
    s = f"b={cfg['b']},h={cfg['h']},m={cfg['m']},n={cfg['n']},d={cfg['d']},is_causal={cfg['is_causal']}"
    if "tag" in cfg:
        s = f"{cfg['tag']}: {s},{cfg['reduction']}"
    return s


def run_row(cfg, ref, want_naive: bool, slice_m: bool, seconds: float, dev, want_cpu: bool = False) -> dict:
    b, h, m, n, d, causal = cfg["b"], cfg["h"], cfg["m"], cfg["n"], cfg["d"], cfg["is_causal"]
    red = cfg.get("reduction", "sum")
    q = torch.randn(b, h, m, d, device=dev, dtype=torch.float16)
    k = torch.randn(b, h, n, d, device=dev, dtype=torch.float16)
    scores = valid_scores(b, h, m, n, causal)
    ours = lambda: chunked_call(flash_colreduce, q, k, red, causal)
    lat = measure_latency(ours, seconds=seconds)
    row = dict(config=_label(cfg), ours_ms=lat * 1e3, ours_mb=measure_memory(ours) / 2**20,
               gscores_per_s=scores / lat / 1e9, tflops=4 * d * scores / lat / 1e12)
    if ref is not None:
        try:
            theirs = lambda: chunked_call(ref.flash_colreduce, q, k, red, causal)
            got, want = ours().float(), theirs().float()
            row["max_abs_diff_vs_reference"] = float((got - want).abs().max())
            rlat = measure_latency(theirs, seconds=seconds)
            row.update(reference_ms=rlat * 1e3, reference_mb=measure_memory(theirs) / 2**20, speedup_vs_reference=rlat / lat)
        except Exception as exc:  # the table keeps the error text in place of a number
            row["reference_error"] = f"{type(exc).__name__}: {exc}"[:200]
    if want_naive and b * h * m * n <= 2**35:
        # the reference's own definition when it was loaded, else this package's restatement of it
        naive_op = ref.naive_colreduce if ref is not None else naive_colreduce
        naive = lambda: chunked_call(naive_op, q, k, red, causal)
        nlat = measure_latency(naive, min_iters=3, seconds=min(seconds, 0.5))
        row.update(naive_ms=nlat * 1e3, naive_mb=measure_memory(naive) / 2**20, speedup_vs_naive=nlat / lat)
    if want_cpu and "tag" in cfg and b * h * m * n <= 2**35:
        ms, threads, how = cpu_definition_ms(cfg, ref, q, k, red)
        row.update(cpu_ms=ms, cpu_threads=threads, cpu_how=how, speedup_vs_cpu=ms / (lat * 1e3))
    if slice_m and m >= 512:
        # the same rows as two query-row slices of a tensor twice as long: non-contiguous views
        big = torch.randn(b, h, 2 * m, d, device=dev, dtype=torch.float16)
        row["ours_sliced_ms"] = measure_latency(
            lambda: flash_colreduce(big[:, :, m // 2: m // 2 + m], k, red, is_causal=causal), seconds=seconds) * 1e3
        del big
    del q, k
    return row


def cpu_definition_ms(cfg, ref, q, k, red):
    """The materialising definition on the host cores in fp32 (all threads), as a reported baseline:
    median of five calls after a warm-up for problems of up to 2^28 scores, else eight (batch, head)
    pairs spread over the problem, one at a time, scaled to all of them (labelled as extrapolated)."""
    import os

    torch.set_num_threads(os.cpu_count() or 1)
    op = ref.naive_colreduce if ref is not None else naive_colreduce
    b, h, m, n = cfg["b"], cfg["h"], cfg["m"], cfg["n"]
    qc, kc = q.float().cpu(), k.float().cpu()
    if b * h * m * n <= 2**28:
        op(qc, kc, reduction=red, is_causal=cfg["is_causal"])
        times = []
        for _ in range(5):
            t0 = time.perf_counter()
            op(qc, kc, reduction=red, is_causal=cfg["is_causal"])
            times.append(time.perf_counter() - t0)
        return sorted(times)[2] * 1e3, torch.get_num_threads(), "whole problem, median of 5"
    pairs = [(i * b * h) // 8 for i in range(8)]
    t0 = time.perf_counter()
    for bh in pairs:
        bi, hi = divmod(bh, h)
        op(qc[bi:bi + 1, hi:hi + 1], kc[bi:bi + 1, hi:hi + 1], reduction=red, is_causal=cfg["is_causal"])
    per_head = (time.perf_counter() - t0) / len(pairs)
    return per_head * b * h * 1e3, torch.get_num_threads(), f"extrapolated from {len(pairs)} of {b * h} heads"


def _fmt(row, key, spec="{:.3f}"):
    return spec.format(row[key]) if key in row else "-"


def to_markdown(rows, gpu: str) -> str:
    head = ("| configuration | this library ms | reference (Triton) ms | speed-up vs reference | naive ms | speed-up vs naive | "
            "this MB | reference MB | naive MB | Gscores/s | TFLOP/s | max abs diff vs reference | definition on host cores ms |")
    lines = [f"GPU: {gpu}", "", head, "|" + "---|" * 13]
    for r in rows:
        ref_ms = _fmt(r, "reference_ms") if "reference_error" not in r else r["reference_error"]
        lines.append(
            f"| {r['config']} | {r['ours_ms']:.3f} | {ref_ms} | {_fmt(r, 'speedup_vs_reference', '{:.2f}')} | "
            f"{_fmt(r, 'naive_ms')} | {_fmt(r, 'speedup_vs_naive', '{:.2f}')} | {r['ours_mb']:.1f} | "
            f"{_fmt(r, 'reference_mb', '{:.1f}')} | {_fmt(r, 'naive_mb', '{:.1f}')} | {r['gscores_per_s']:.1f} | "
            f"{r['tflops']:.1f} | {_fmt(r, 'max_abs_diff_vs_reference', '{:.2e}')} | "
            + (f"{r['cpu_ms']:.1f} ({r['cpu_threads']} threads, {r['cpu_how']})" if "cpu_ms" in r else "-") + " |")
    return "\n".join(lines) + "\n"


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference-path", default=None,
                    help="directory holding the unmodified reference package `flash_colreduce` (timed beside this library)")
    ap.add_argument("--naive", action="store_true", help="also time the materialising definition on the GPU")
    ap.add_argument("--configs", action="store_true", help="append the metric's own configurations")
    ap.add_argument("--only-configs", action="store_true", help="skip the 20 shapes")
    ap.add_argument("--slice-m", action="store_true", help="also time this library on query-row slices (strided views)")
    ap.add_argument("--cpu", action="store_true",
                    help="also time the materialising definition on the host cores for the metric's configurations")
    ap.add_argument("--seconds", type=float, default=1.0, help="length of each warm-up and each timed run")
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None)
    args = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    gpu = torch.cuda.get_device_name(dev)
    ref = _load_reference(args.reference_path) if args.reference_path else None
    print(f"GPU: {gpu}" + (f"; reference {getattr(ref, '__version__', '?')} from {args.reference_path}" if ref else ""))
    shapes = ([] if args.only_configs else list(SHAPES)) + (list(METRIC_CONFIGS) if args.configs or args.only_configs else [])
    rows = []
    for cfg in shapes:
        row = run_row(cfg, ref, args.naive, args.slice_m, args.seconds, dev, args.cpu)
        print(json.dumps(row), flush=True)
        rows.append(row)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    if args.md:
        with open(args.md, "w") as f:
            f.write(to_markdown(rows, gpu))


if __name__ == "__main__":
    main()
