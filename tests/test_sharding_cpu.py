"""Multi-rank host logic on CPU ranks (gloo, world size 2 and 4): shard plans and the reduce."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flash_colreduce_b200.sharding import plan_shards, sharded_colreduce
from oracle import oracle_colreduce


def test_head_partition_is_exact():
    for bh, world in ((64, 8), (7, 3), (8, 8), (130, 4)):
        seen = []
        for r in range(world):
            s = plan_shards(bh, 1000, world, r)
            assert not s.needs_reduce and s.row_ranges == [(0, 1000)]
            seen += list(range(s.head_lo, s.head_hi))
        assert seen == list(range(bh))


def test_row_split_covers_rows_once_and_balances_causal_work():
    m = 131072
    for bh, world in ((1, 8), (2, 8), (4, 8), (1, 2), (3, 8)):
        per_head = {}
        for r in range(world):
            s = plan_shards(bh, m, world, r)
            assert s.needs_reduce
            if s.heads == 0:
                continue
            per_head.setdefault(s.head_lo, []).extend(s.row_ranges)
        assert sorted(per_head) == list(range(bh))
        for ranges in per_head.values():
            rows = sorted(ranges)
            assert rows[0][0] == 0 and rows[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(rows, rows[1:]))
        # causal work of a row ~ its index: zig-zag keeps ranks within 1% of each other
        work = []
        for r in range(world):
            s = plan_shards(bh, m, world, r)
            if s.heads:
                work.append(sum((hi * (hi + 1) - lo * (lo + 1)) // 2 for lo, hi in s.row_ranges))
        assert max(work) <= 1.01 * min(work)


def test_c_shard_plan_is_the_same_rule():
    """fcr_plan_shards (what fcr_colreduce_sharded runs on) against the Python planner."""
    from flash_colreduce_b200.sharding import native_plan_shards

    for bh in (1, 2, 3, 7, 8, 64):
        for m in (1, 128, 129, 3000, 131072):
            for world in (1, 2, 3, 4, 8):
                for rank in range(world):
                    a, b = plan_shards(bh, m, world, rank), native_plan_shards(bh, m, world, rank)
                    assert (a.head_lo, a.head_hi, a.row_ranges, a.needs_reduce) == (b.head_lo, b.head_hi, b.row_ranges, b.needs_reduce)
    with pytest.raises(ValueError):
        native_plan_shards(4, 10, 2, 2)


def test_sharded_entry_rejects_bad_arguments_before_any_device_work():
    import ctypes as C

    from flash_colreduce_b200 import _native as nat

    prob = nat.make_problem(1, 2, 256, 256, 64, (2 * 256 * 64, 256 * 64, 64, 1), (2 * 256 * 64, 256 * 64, 64, 1), nat.FCR_F16,
                            nat.FCR_SUM, True, 0.125)
    sh = nat.Shard()
    assert nat.lib.fcr_plan_shards(2, 256, 1, 0, C.byref(sh)) == nat.FCR_OK
    call = lambda p, s, heads, acc, out: nat.lib.fcr_colreduce_sharded(p, s, heads, None, None, acc, out, nat.FCR_F16, None, 0, None, None)
    assert call(None, C.byref(sh), 2, None, None) == nat.FCR_ERR_BAD_ARG
    assert call(C.byref(prob), C.byref(sh), 2, None, None) == nat.FCR_ERR_BAD_ARG and "null acc" in nat.last_error()
    sh.row_hi[0] = 300  # beyond M
    assert call(C.byref(prob), C.byref(sh), 2, None, None) == nat.FCR_ERR_BAD_ARG and "row range" in nat.last_error()
    sh.row_hi[0] = 256
    sh.head_hi = 3      # three heads against a two-head local problem
    assert call(C.byref(prob), C.byref(sh), 3, None, None) == nat.FCR_ERR_BAD_ARG and "exactly the shard's heads" in nat.last_error()
    assert nat.lib.fcr_comm_init(None, 2, 0, None) == nat.FCR_ERR_BAD_ARG
    assert nat.lib.fcr_comm_destroy(None) == nat.FCR_OK


def test_bad_arguments():
    with pytest.raises(ValueError):
        plan_shards(4, 10, 2, 2)
    with pytest.raises(ValueError):
        plan_shards(0, 10, 2, 0)


def _cpu_partial(q, k, reduction, is_causal, scale, causal_offset):
    """Oracle for a row slice whose row i attends keys j <= i + causal_offset.

    The oracle aligns its mask as max(N - M, 0); embedding the slice after
    ``causal_offset`` zero rows in a problem with at least N rows makes that
    alignment 0, so that embedded row causal_offset + i attends keys <= causal_offset + i.
    """
    m_rows = q.shape[2]
    n = k.shape[2]
    if not is_causal:
        return oracle_colreduce(q, k, reduction, False, scale)
    pre = causal_offset
    tail = max(0, n - (pre + m_rows))
    zeros = lambda r: torch.zeros(q.shape[0], q.shape[1], r, q.shape[3], dtype=q.dtype)
    q_ext = torch.cat([zeros(pre), q, zeros(tail)], dim=2)
    return oracle_colreduce(q_ext, k, reduction, True, scale, row_range=(pre, pre + m_rows), apply_mean=False)


def _cpu_finalize(acc, m, reduction, is_causal, dtype):
    b, h, n = acc.shape
    out = acc.clone()
    if reduction == "mean":
        if is_causal:
            c = max(n - m, 0)
            out[..., :c] /= m
            out[..., c:] /= torch.arange(n - c, 0, -1).float()
        else:
            out /= m
    return out.to(dtype)


def _worker(rank, world, port, bh, m, n, causal, reduction, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        q = torch.randn(1, bh, m, 16, generator=g)
        k = torch.randn(1, bh, n, 16, generator=g)
        spec = plan_shards(bh, m, world, rank)
        out = sharded_colreduce(q[:, spec.head_lo:spec.head_hi], k[:, spec.head_lo:spec.head_hi], reduction, causal,
                                spec=spec, total_heads=bh, partial_fn=_cpu_partial, finalize_fn=_cpu_finalize)
        want = oracle_colreduce(q, k, reduction, causal)[0]
        torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-6)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,bh,m,n,causal,reduction", [
    (2, 4, 300, 300, True, "sum"),     # heads partitioned
    (2, 1, 700, 900, True, "mean"),    # rows of one head split over both ranks, M < N
    (2, 1, 515, 260, True, "max"),     # M > N
    (4, 2, 1024, 1024, True, "sum"),   # two ranks per head
    (2, 1, 400, 300, False, "mean"),
])
def test_sharded_result_equals_single_process(tmp_path, world, bh, m, n, causal, reduction):
    mp.spawn(_worker, args=(world, _free_port(), bh, m, n, causal, reduction, str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == [f"ok{r}" for r in range(world)]
