"""A device-side wait that runs out is reported to the host (needs a B200).

The failure is made without faulting anything: a self-test hook makes the first
CTA of each pass kernel leave out one streamed-tile load (nothing is in flight
for that slot) and shortens the bound of every device-side wait to about a
millisecond.  The waits on the missing tile then expire, every warp of that CTA
leaves through the kernel's normal give-up path (tensor memory released), the
kernels return, and the status reaches the host through the mailbox in mapped
host memory -- no synchronisation needed by the library to notice it.
"""
import ctypes as C
import math
import os

import pytest
import torch

from conftest import assert_parity
from oracle import oracle_colreduce

pytestmark = pytest.mark.gpu

ST_WAIT_RING_FULL, ST_WAIT_TMEM_FULL = 22, 31  # the MMA warps' wait on the tile, the softmax warps' on its product


@pytest.fixture
def no_debug_sync():
    old = os.environ.get("FCR_DEBUG_SYNC")
    os.environ["FCR_DEBUG_SYNC"] = "0"  # the point is that nobody synchronises to read status words
    yield
    if old is None:
        os.environ.pop("FCR_DEBUG_SYNC", None)
    else:
        os.environ["FCR_DEBUG_SYNC"] = old


def _inputs(dev):
    g = torch.Generator().manual_seed(5)
    # 64 heads x 4 row blocks = 256 work items on 148 SMs: no split, every item streams 32 key tiles
    q = torch.randn(1, 64, 1024, 128, generator=g).half()
    k = torch.randn(1, 64, 4096, 128, generator=g).half()
    return q, k, q.to(dev), k.to(dev)


def test_expired_wait_reaches_the_host_through_the_mailbox(no_debug_sync):
    from flash_colreduce_b200 import _native as nat
    from flash_colreduce_b200 import flash_colreduce

    dev = torch.device("cuda:0")
    q, k, qd, kd = _inputs(dev)
    flash_colreduce(qd, kd, "sum")  # normal call first: creates the mailbox, proves the shape runs
    torch.cuda.synchronize()
    code = C.c_int32(-1)
    assert nat.lib.fcr_poll_device_status(C.byref(code)) == nat.FCR_OK and code.value == 0

    nat.check(nat.lib.fcr_self_test_hooks(2_000_000, 2), "fcr_self_test_hooks")  # ~1 ms; third load of CTA 0 left out
    try:
        flash_colreduce(qd, kd, "sum")  # launches fine; the kernels give up on the device
    finally:
        nat.check(nat.lib.fcr_self_test_hooks(0, -1), "fcr_self_test_hooks")
    torch.cuda.synchronize()  # the test waits for the kernels; the library does not need to
    rc = nat.lib.fcr_poll_device_status(C.byref(code))
    assert rc == nat.FCR_ERR_DEVICE_TIMEOUT
    assert code.value in (ST_WAIT_RING_FULL, ST_WAIT_TMEM_FULL), nat.last_error()
    assert "block 0" in nat.last_error() and "bounded wait" in nat.last_error()
    assert nat.lib.fcr_poll_device_status(C.byref(code)) == nat.FCR_OK  # reported once

    # the context is intact: the same call now succeeds and is right
    got = flash_colreduce(qd, kd, "sum")
    want = oracle_colreduce(q[:, :2], k[:, :2], "sum", False)
    assert_parity(got[:, :2], want, "sum", extra_rtol=2.0 ** -11)


def test_the_next_call_raises_for_the_failed_one(no_debug_sync):
    from flash_colreduce_b200 import _native as nat
    from flash_colreduce_b200 import flash_colreduce

    dev = torch.device("cuda:0")
    _, _, qd, kd = _inputs(dev)
    flash_colreduce(qd, kd, "max", is_causal=True)
    nat.check(nat.lib.fcr_self_test_hooks(2_000_000, 1), "fcr_self_test_hooks")
    try:
        flash_colreduce(qd, kd, "max", is_causal=True)
    finally:
        nat.check(nat.lib.fcr_self_test_hooks(0, -1), "fcr_self_test_hooks")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="status 4.*earlier call"):
        flash_colreduce(qd, kd, "max", is_causal=True)
    out = flash_colreduce(qd, kd, "max", is_causal=True)  # and the one after that runs
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()


def test_status_words_in_the_workspace_tell_the_same_story():
    """fcr_read_device_status (synchronising) on the workspace of the failed call."""
    from flash_colreduce_b200 import _native as nat

    dev = torch.device("cuda:0")
    _, _, qd, kd = _inputs(dev)
    b, h, m, d = qd.shape
    n = kd.shape[2]
    prob = nat.make_problem(b, h, m, n, d, qd.stride(), kd.stride(), nat.FCR_F16, nat.FCR_SUM, False, 1 / math.sqrt(d))
    pl = nat.plan(prob, 0)
    ws = torch.empty(int(pl.workspace_bytes), dtype=torch.uint8, device=dev)
    out = torch.empty((b, h, n), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    nat.check(nat.lib.fcr_self_test_hooks(2_000_000, 2), "fcr_self_test_hooks")
    try:
        nat.check(nat.lib.fcr_colreduce(C.byref(prob), qd.data_ptr(), kd.data_ptr(), out.data_ptr(), nat.FCR_F32,
                                        ws.data_ptr(), ws.numel(), stream), "fcr_colreduce")
    finally:
        nat.check(nat.lib.fcr_self_test_hooks(0, -1), "fcr_self_test_hooks")
    code = C.c_int32(0)
    assert nat.lib.fcr_read_device_status(ws.data_ptr(), stream, C.byref(code)) == nat.FCR_ERR_DEVICE_TIMEOUT
    assert code.value in (ST_WAIT_RING_FULL, ST_WAIT_TMEM_FULL)
    # that read also took the report out of the mailbox
    assert nat.lib.fcr_poll_device_status(C.byref(code)) == nat.FCR_OK
