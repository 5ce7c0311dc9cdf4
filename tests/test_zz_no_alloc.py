"""The allocation-free entry point, checked against the regular one and the oracle
(needs a B200; collected last on purpose).

``fcr_colreduce_static`` serves hosts that cannot allocate device memory where
the library runs -- a plugin inside another runtime's enqueue hook, a process
whose device memory all belongs to one arena -- by keeping the kernels' scratch
in a fixed array inside the library image.  The array is shared by every call
and keeps the previous call's contents, so the check is done several times in a
row, with different problems, through the C ABI: the results must be bit-for-bit
those of ``fcr_colreduce`` (same kernels, same plan), within the parity bar of
the oracle, and the device's free memory must not move.
"""
import ctypes as C
import math

import pytest
import torch

from conftest import assert_parity
from oracle import oracle_colreduce

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 8 << 20  # FCR_STATIC_SCRATCH_BYTES in include/flash_colreduce_b200.h


def _run_both(nat, q, k, reduction, causal):
    """Returns (regular entry point result, allocation-free entry point result, plan), results in fp32."""
    b, h, m, d = q.shape
    n = k.shape[2]
    prob = nat.make_problem(b, h, m, n, d, q.stride(), k.stride(), nat.FCR_F16, nat.REDUCTION_CODES[reduction], causal,
                            1 / math.sqrt(d))
    pl = nat.plan(prob, 0)
    assert pl.workspace_bytes <= STATIC_SCRATCH_BYTES
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(int(pl.workspace_bytes), dtype=torch.uint8, device=q.device)
    want = torch.empty((b, h, n), dtype=torch.float32, device=q.device)
    nat.check(nat.lib.fcr_colreduce(C.byref(prob), q.data_ptr(), k.data_ptr(), want.data_ptr(), nat.FCR_F32,
                                    ws.data_ptr(), ws.numel(), stream), "fcr_colreduce")
    got = torch.full((b, h, n), float("nan"), dtype=torch.float32, device=q.device)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(q.device)[0]
    nat.check(nat.lib.fcr_colreduce_static(C.byref(prob), q.data_ptr(), k.data_ptr(), got.data_ptr(), nat.FCR_F32,
                                           stream), "fcr_colreduce_static")
    code = C.c_int32(-1)
    nat.check(nat.lib.fcr_read_device_status_static(stream, C.byref(code)), "fcr_read_device_status_static")
    assert code.value == 0
    free_after = torch.cuda.mem_get_info(q.device)[0]
    return want, got, pl, free_before - free_after


def test_static_scratch_entry_point_matches_regular_entry_point_and_oracle():
    from flash_colreduce_b200 import _native as nat

    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(42)
    # first call: a decode-like shape whose key range is split, so the scratch holds split partials
    q1 = torch.randn(1, 4, 128, 128, generator=g).half()
    k1 = torch.randn(1, 4, 2048, 128, generator=g).half()
    want, got, pl, _ = _run_both(nat, q1.to(dev), k1.to(dev), "mean", True)  # first call on the device: address look-up
    assert pl.row_splits > 1
    assert torch.equal(got, want)
    assert_parity(got, oracle_colreduce(q1, k1, "mean", True), "mean")
    # second call right after it: another shape and reduction over the scratch the first call left behind
    q2 = torch.randn(2, 3, 700, 64, generator=g).half()
    k2 = torch.randn(2, 3, 333, 64, generator=g).half()
    want, got, _, grew = _run_both(nat, q2.to(dev), k2.to(dev), "max", True)
    assert torch.equal(got, want) and grew == 0, f"free device memory changed by {grew} bytes"
    assert_parity(got, oracle_colreduce(q2, k2, "max", True), "max")
    want, got, _, grew = _run_both(nat, q1.to(dev), k1.to(dev), "sum", False)
    assert torch.equal(got, want) and grew == 0
    assert_parity(got, oracle_colreduce(q1, k1, "sum", False), "sum")
    # decode with a handful of queries: the score cache lies inside the array too
    q3 = torch.randn(2, 4, 8, 128, generator=g).half()
    k3 = torch.randn(2, 4, 4096, 128, generator=g).half()
    want, got, pl, grew = _run_both(nat, q3.to(dev), k3.to(dev), "sum", True)
    assert pl.score_cache == 1 and pl.off_scores > 0 and pl.workspace_bytes <= STATIC_SCRATCH_BYTES
    assert torch.equal(got, want) and grew == 0
    assert_parity(got, oracle_colreduce(q3, k3, "sum", True), "sum")


def test_static_scratch_rejects_problems_beyond_its_size():
    from flash_colreduce_b200 import _native as nat

    dev = torch.device("cuda:0")
    q = torch.zeros(1, 8, 131072 * 2, 64, dtype=torch.float16, device=dev)  # 8 heads x 262144 rows of lse = 8 MiB + status
    prob = nat.make_problem(1, 8, q.shape[2], q.shape[2], 64, q.stride(), q.stride(), nat.FCR_F16, nat.FCR_SUM, True, 0.125)
    assert nat.lib.fcr_workspace_bytes(C.byref(prob), 0) > STATIC_SCRATCH_BYTES
    out = torch.zeros(1, 8, q.shape[2], dtype=torch.float32, device=dev)
    rc = nat.lib.fcr_colreduce_static(C.byref(prob), q.data_ptr(), q.data_ptr(), out.data_ptr(), nat.FCR_F32,
                                      torch.cuda.current_stream().cuda_stream)
    assert rc == nat.FCR_ERR_WORKSPACE
    assert "built-in scratch holds 8388608" in nat.last_error()
