"""Benchmark of the column-reduction hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload msplit]

One step = one pass of ``flash_colreduce`` over the long-context workload
(B=1, H=64, M=N=131072, d=128, fp16, causal, reduction "sum").  With N GPUs the
64 heads are partitioned over the ranks (no data-path collective: heads are
independent), so the job is strong-scaled.  The line printed by rank 0 reports
attention scores reduced per second, the tensor-core roofline of the two QK^T
passes, the same metric end to end from pinned host buffers, a CPU baseline
and, on one GPU, the reference's own Triton kernel timed on the same inputs.

``--workload msplit`` measures the other way the operator shards: fewer heads
than GPUs (max(1, N/2) heads of the same 131072-square problem, two ranks per
head from N = 2 on), the query rows of a head split zig-zag over its ranks and
the partial column vectors combined by one NCCL all-reduce.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(B=1, H=64, M=131072, N=131072, D=128, causal=True, reduction="sum")
METRIC = "attn_scores_reduced_per_s"
UNIT = "scores/s"
# DRAM bytes (read + write) of one pass-kernel launch per byte of Q and K it is given, measured with ncu on a
# two-head slice of this workload (same 64 MiB heads, same interleaving of two heads; profiles/): the
# re-streaming of the operands is served by the L2 (98 % hits), part of a head is read from DRAM more than once.
TRAFFIC_PER_INPUT_BYTE = {"rows": 1.553, "cols": 1.268}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["bf16_tflops_sustained"]), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz, self.power = [], set(), None, []
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
                except Exception:
                    pass
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        s = sorted(self.samples)
        w = sorted(self.power)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "power_w": w[len(w) // 2] if w else None}


def _use_all_host_threads() -> int:
    """The CPU legs use every host core: a launcher such as torchrun exports OMP_NUM_THREADS=1."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return torch.get_num_threads()


def _cpu_baseline(seconds: float, steps: int | None = None, warmup: int = 0):
    """Times the CPU oracle (the port of the reference's naive_colreduce) on a bounded sample.

    Sample: one head of the workload, 8 blocks of 256 query rows centred in 8 equal
    segments of the M rows (so the masked fraction matches the whole problem's),
    each block against all N keys, exactly as the materialising definition does.
    Returns (scores per second, threads, description, seconds per step).
    """
    from oracle import oracle_colreduce

    _use_all_host_threads()
    w = WORKLOAD
    m, n, d = w["M"], w["N"], w["D"]
    g = torch.Generator().manual_seed(0)
    k = torch.randn(1, 1, n, d, generator=g).half().float()
    rows_per_block, segments = 256, 8
    blocks = []
    for s in range(segments):
        centre = (2 * s + 1) * m // (2 * segments)
        blocks.append((centre - rows_per_block // 2, centre + rows_per_block // 2))
    # rows [lo, hi) of the full problem: each block is embedded in an M-row tensor so that the oracle's
    # right-aligned mask gives row lo + i the keys 0 .. lo + i (built once, outside the timed steps)
    q_exts = []
    for lo, hi in blocks:
        q_ext = torch.zeros(1, 1, m, d)
        q_ext[:, :, lo:hi] = torch.randn(1, 1, hi - lo, d, generator=g).half().float()
        q_exts.append(q_ext)
    scores_per_step = sum(sum(min(i + 1, n) for i in range(lo, hi)) for lo, hi in blocks)
    scale = d ** -0.5

    def step():
        for (lo, hi), q_ext in zip(blocks, q_exts):  # the definition materialises all N keys for every row
            oracle_colreduce(q_ext, k, "sum", True, scale, row_range=(lo, hi), block_rows=rows_per_block)

    for _ in range(warmup):
        step()
    times = []
    t_start = time.perf_counter()
    while True:
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
        if steps is not None:
            if len(times) >= steps:
                break
        elif time.perf_counter() - t_start >= seconds and len(times) >= 3:
            break
    total = sum(times)
    sample = (f"one head of the workload: {segments} blocks of {rows_per_block} query rows centred in {segments} equal "
              f"segments of M, each against all N keys in fp32 ({scores_per_step} valid scores per step), "
              f"{len(times)} steps, {total:.1f} s")
    return scores_per_step * len(times) / total, torch.get_num_threads(), sample, total / len(times)


def run_reference(args):
    """The reference arm: the reference's CPU implementation of the path (its materialising
    definition, restated in oracle/) on all host cores, on a bounded sample of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, cores, sample, sec_per_step = _cpu_baseline(0.0, steps=args.steps, warmup=args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "long-context B=1 H=64 M=N=131072 d=128 causal sum (bounded sample per step)", **WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class _Dist:
    """Rank bookkeeping and the few collectives the benchmark itself needs."""

    def __init__(self, args):
        import torch.distributed as dist

        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group("nccl", device_id=self.dev)

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, x: float, op: str) -> float:
        if self.world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        ops = {"max": self.dist.ReduceOp.MAX, "min": self.dist.ReduceOp.MIN, "sum": self.dist.ReduceOp.SUM}
        self.dist.all_reduce(t, op=ops[op])
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def _head_inputs(dev, heads, M, N, D):
    """fp16 N(0,1) inputs, one seed per global head index so that shards do not depend on the GPU count."""
    q = torch.empty((1, len(heads), M, D), dtype=torch.float16, device=dev)
    k = torch.empty((1, len(heads), N, D), dtype=torch.float16, device=dev)
    gen = torch.Generator(device=dev)
    for i, bh in enumerate(heads):
        gen.manual_seed(bh)
        q[0, i] = torch.randn((M, D), generator=gen, device=dev, dtype=torch.float32).half()
        k[0, i] = torch.randn((N, D), generator=gen, device=dev, dtype=torch.float32).half()
    return q, k


def _reference_gpu(q, k, total_scores, path):
    """The unmodified reference package (its Triton kernel, JIT-compiled here) on the same device
    tensors: a baseline beside the product, imported only by this function."""
    info = {"path": path}
    try:
        sys.path.insert(0, path)
        try:
            import flash_colreduce as ref
        finally:
            sys.path.remove(path)
        ref.flash_colreduce(q, k, reduction="sum", is_causal=True)  # compiles
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 2
        e0.record()
        for _ in range(reps):
            out = ref.flash_colreduce(q, k, reduction="sum", is_causal=True)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        info.update(version=getattr(ref, "__version__", None), ms_per_step=ms, value=total_scores / (ms * 1e-3), unit=UNIT,
                    steps=reps, checksum=float(out.float().sum().item()),
                    note="reference flash_colreduce (Triton, stock code path) on this GPU, same device-resident inputs")
    except Exception as exc:
        info["unavailable"] = f"{type(exc).__name__}: {exc}"[:300]
    return info


def run_ours(args):
    from flash_colreduce_b200 import _native as nat
    from flash_colreduce_b200 import flash_colreduce, flash_colreduce_host, valid_scores
    from flash_colreduce_b200.ex2_probe import ex2_rate
    from flash_colreduce_b200.sharding import plan_shards

    dd = _Dist(args)
    world, rank, dev = dd.world, dd.rank, dd.dev
    w = WORKLOAD
    B, H, M, N, D = w["B"], w["H"], w["M"], w["N"], w["D"]
    spec = plan_shards(B * H, M, world, rank)
    heads = spec.heads
    assert not spec.needs_reduce, "the benchmark workload has at least one head per GPU"
    total_scores = valid_scores(B, H, M, N, True)
    q, k = _head_inputs(dev, range(spec.head_lo, spec.head_hi), M, N, D)

    def step():
        return flash_colreduce(q, k, "sum", is_causal=True)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        out = step()
    dd.barrier()
    # ---- device-resident throughput: K steps between two events, per-pass times traced live
    nat.lib.fcr_trace_enable(1)
    launches0 = nat.lib.fcr_launch_count()
    with ClockSampler(dd.local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = step()
        e1.record()
        dd.barrier()
    launches = int(dd.reduce(float(nat.lib.fcr_launch_count() - launches0), "sum"))
    ms_total = dd.reduce(e0.elapsed_time(e1), "max")
    passes = nat.trace_times()
    nat.lib.fcr_trace_enable(0)
    ms_step = ms_total / args.steps
    value = total_scores / (ms_step * 1e-3)
    checksum = float(out.float().sum().item())  # column sums add up to the number of rows per head

    ref_gpu = None
    ref_path = os.path.join(ROOT, "baseline", "_ref")
    if world == 1 and not args.no_reference_gpu:
        ref_gpu = (_reference_gpu(q, k, total_scores, ref_path) if os.path.isdir(os.path.join(ref_path, "flash_colreduce"))
                   else {"unavailable": "baseline/_ref holds no reference install"})

    # ---- end to end from pinned host buffers (H2D of q and k, kernels, D2H of the result, every step)
    qh = torch.empty(q.shape, dtype=q.dtype, pin_memory=True).copy_(q)
    kh = torch.empty(k.shape, dtype=k.dtype, pin_memory=True).copy_(k)
    oh = torch.empty((1, heads, N), dtype=q.dtype, pin_memory=True)
    del q, k
    torch.cuda.empty_cache()
    e2e_steps = args.steps
    for _ in range(2):
        flash_colreduce_host(qh, kh, "sum", is_causal=True, device=dev, out=oh)
    dd.barrier()
    t0 = time.perf_counter()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(e2e_steps):
        flash_colreduce_host(qh, kh, "sum", is_causal=True, device=dev, out=oh)
    a1.record()
    torch.cuda.synchronize()
    e2e_ms = dd.reduce(max(a0.elapsed_time(a1), (time.perf_counter() - t0) * 1e3), "max") / e2e_steps
    e2e_value = total_scores / (e2e_ms * 1e-3)
    host_checksum = float(oh.float().sum().item())

    if rank == 0:
        peak_burst, peak_sustained, peak_kind = _peaks()
        rows_ms = sum(p[0] for p in passes) / max(len(passes), 1)
        cols_ms = sum(p[1] for p in passes) / max(len(passes), 1)
        local_scores = total_scores * heads // (B * H)
        # each pass is one QK^T: 2*D flops per valid score; the dominant kernel is the slower pass
        dom_ms = max(rows_ms, cols_ms)
        achieved = 2 * D * local_scores / (dom_ms * 1e-3) / 1e12
        rate = ex2_rate(3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": "long-context B=1 H=64 M=N=131072 d=128 fp16 causal sum, heads partitioned over GPUs",
                       **WORKLOAD, "heads_per_gpu": heads, "l2": "inputs (4 GiB per 64 heads) exceed the 126 MB L2"},
            "roofline": {
                "bound": "tensor", "achieved": achieved, "peak": peak_sustained, "unit": "TFLOP/s",
                "frac": achieved / peak_sustained,
                # DRAM bytes of one pass launch per byte of Q and K, from an ncu capture of a two-head slice of
                # this workload (64 MiB heads, as here); the traffic grows with the heads a rank holds
                "traffic": int(TRAFFIC_PER_INPUT_BYTE["rows" if rows_ms >= cols_ms else "cols"] * 2 * heads * (M + N) * D),
                "algorithmic_flops_per_score_per_launch": 2 * D, "peak_kind": f"{peak_kind} sustained bf16 (kernel timed inside a long step)",
                "kernel": "pass_kernel (rows pass)" if rows_ms >= cols_ms else "pass_kernel (columns pass)",
                "rows_pass_ms": rows_ms, "cols_pass_ms": cols_ms,
                "op_tflops": 4 * D * local_scores / ((rows_ms + cols_ms) * 1e-3) / 1e12,
                "op_frac_of_burst_peak": 4 * D * local_scores / ((rows_ms + cols_ms) * 1e-3) / 1e12 / peak_burst,
                "exp_rate_measured": rate,
                "exp_bound_frac": (local_scores / rate) / ((rows_ms + cols_ms) * 1e-3) if rate else None,
            },
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(qh.numel() + kh.numel()) * 2 * world,
                    "d2h_bytes_per_step": int(oh.numel()) * 2 * world, "ms_per_step": e2e_ms, "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
            "checksum": {"device": checksum, "host": host_checksum, "expected": float(heads * M)},
        }
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        if world == 1 and not args.no_cpu_baseline:
            v, cores, sample, _ = _cpu_baseline(12.0)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    dd.close()


def run_msplit(args):
    """Fewer heads than GPUs: the rows of a head are split over its ranks, one all-reduce combines."""
    from flash_colreduce_b200 import _native as nat
    from flash_colreduce_b200 import colreduce_partial, valid_scores
    from flash_colreduce_b200.sharding import NativeComm, plan_shards, sharded_colreduce, sharded_colreduce_native

    dd = _Dist(args)
    world, rank, dev = dd.world, dd.rank, dd.dev
    M = N = WORKLOAD["M"]
    D = WORKLOAD["D"]
    H = max(1, world // 2)  # two ranks per head from two GPUs on: the work per GPU stays the same
    spec = plan_shards(H, M, world, rank)
    total_scores = valid_scores(1, H, M, N, True)
    q, k = _head_inputs(dev, range(spec.head_lo, spec.head_hi), M, N, D)
    scale = D ** -0.5

    # the library's own multi-GPU entry (fcr_colreduce_sharded) on a communicator it made itself
    comm = NativeComm() if world > 1 else None

    def step(reduction="sum"):
        return sharded_colreduce_native(q, k, reduction, True, scale, total_heads=H, comm=comm, world=world, rank=rank)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        out = step()
    dd.barrier()
    launches0 = nat.lib.fcr_launch_count()
    with ClockSampler(dd.local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = step()
        e1.record()
        dd.barrier()
    launches = int(dd.reduce(float(nat.lib.fcr_launch_count() - launches0), "sum"))
    ms_step = dd.reduce(e0.elapsed_time(e1), "max") / args.steps

    # ---- this rank's kernels alone (no collective), for the all-reduce's share and the balance between ranks
    def kernels_only():
        for lo, hi in spec.row_ranges:
            colreduce_partial(q[:, :, lo:hi], k[:, :, :hi], "sum", True, scale, lo)

    kernels_only()
    dd.barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
        kernels_only()
    k1.record()
    torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / args.steps
    kern_max, kern_min = dd.reduce(kern_ms, "max"), dd.reduce(kern_ms, "min")
    # the all-reduce of the fp32 (H, N) array alone
    buf = torch.zeros((1, H, N), dtype=torch.float32, device=dev)
    ar_ms = 0.0
    if world > 1:
        for _ in range(3):
            dd.dist.all_reduce(buf)
        dd.barrier()
        r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        r0.record()
        for _ in range(args.steps):
            dd.dist.all_reduce(buf)
        r1.record()
        torch.cuda.synchronize()
        ar_ms = dd.reduce(r0.elapsed_time(r1) / args.steps, "max")

    # ---- invariance under the shard count: head 0 computed whole on one GPU against the sharded result
    check = {}
    out_max = step("max")
    # the Python driver over torch.distributed (same plan, same kernels) must agree with the C entry
    via_torch = sharded_colreduce(q, k, "max", True, scale, spec=spec, total_heads=H)
    agree = bool(torch.equal(via_torch, out_max))
    if rank == 0:
        from flash_colreduce_b200 import flash_colreduce

        q0, k0_ = _head_inputs(dev, [0], M, N, D)
        whole_sum = flash_colreduce(q0, k0_, "sum", is_causal=True)
        whole_max = flash_colreduce(q0, k0_, "max", is_causal=True)
        rel = ((out[0].float() - whole_sum[0, 0].float()).abs() / whole_sum[0, 0].float().abs().clamp_min(1e-6)).max()
        check = {"max_bitwise_equal_to_one_gpu": bool(torch.equal(out_max[0], whole_max[0, 0])),
                 "max_bitwise_equal_to_torch_distributed_driver": agree,
                 "sum_max_rel_diff_to_one_gpu": float(rel), "column_sums_total": float(out.float().sum().item()),
                 "column_sums_expected": float(H * M)}
    if rank == 0:
        line = {
            "metric": METRIC, "value": total_scores / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp16", "data": "synthetic",
            "config": {"workload": f"row split: B=1 H={H} M=N={M} d={D} fp16 causal sum, {world // H} rank(s) per head, "
                                   "rows cut zig-zag, one all-reduce of the fp32 (H, N) partial sums", "H": H, "M": M, "N": N,
                       "D": D, "ranks_per_head": world // H, "row_ranges_rank0": spec.row_ranges,
                       "l2": "a head's Q and K (64 MiB) fit the L2; every step re-reads them after the all-reduce"},
            "allreduce_ms": ar_ms, "allreduce_share": ar_ms / ms_step if ms_step else None,
            "kernels_ms_max_over_ranks": kern_max, "kernels_ms_min_over_ranks": kern_min,
            "load_imbalance": kern_max / kern_min if kern_min else None,
            "shard_invariance": check, "gpu_launches": launches, "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if comm is not None:
        comm.close()
    dd.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c5", choices=["c5", "msplit"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "msplit":
        run_msplit(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
