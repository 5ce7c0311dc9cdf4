"""The library's multi-GPU entry point (fcr_colreduce_sharded) exercised on ONE GPU.

With a single rank the entry runs its whole queue -- memset, kernels per row range, fold, finalize --
without a communicator.  The shards of a two- and four-rank plan are run one after the other with
their world size set to one (no all-reduce) and added up on the host: that is the row-range code
path of the entry, checked against the oracle.  The real multi-rank runs are in test_gpu_sharded.py.
"""
import ctypes as C
import math

import pytest
import torch

from conftest import assert_parity
from oracle import oracle_colreduce

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("reduction", ["sum", "mean", "max"])
@pytest.mark.parametrize("causal", [False, True])
def test_one_rank_is_bit_for_bit_the_operator(reduction, causal):
    from flash_colreduce_b200 import flash_colreduce
    from flash_colreduce_b200.sharding import sharded_colreduce_native

    g = torch.Generator().manual_seed(17)
    q = torch.randn(1, 5, 700, 64, generator=g).half().to(_dev())
    k = torch.randn(1, 5, 900, 64, generator=g).half().to(_dev())
    got = sharded_colreduce_native(q, k, reduction, causal, total_heads=5, comm=None, world=1, rank=0)
    want = flash_colreduce(q, k, reduction, is_causal=causal)[0]
    assert got.shape == want.shape and got.dtype == want.dtype
    assert torch.equal(got, want)


@pytest.mark.parametrize("world,m,n,causal,reduction", [(2, 3000, 3000, True, "sum"), (4, 2100, 2600, True, "sum"),
                                                        (2, 1500, 520, True, "max"), (4, 1024, 2048, False, "sum")])
def test_row_ranges_of_a_multi_rank_plan_add_up(world, m, n, causal, reduction):
    """Rank by rank on one GPU: each shard's fp32 partial through the C entry, combined on the host."""
    from flash_colreduce_b200 import _native as nat

    dev = _dev()
    g = torch.Generator().manual_seed(world * 100 + m)
    q = torch.randn(1, 1, m, 64, generator=g).half()
    k = torch.randn(1, 1, n, 64, generator=g).half()
    qd, kd = q.to(dev), k.to(dev)
    prob = nat.make_problem(1, 1, m, n, 64, qd.stride(), kd.stride(), nat.FCR_F16, nat.REDUCTION_CODES[reduction], causal,
                            1 / math.sqrt(64))
    stream = torch.cuda.current_stream().cuda_stream
    total = torch.zeros(1, n, dtype=torch.float32, device=dev)
    rows_seen = 0
    for rank in range(world):
        sh = nat.Shard()
        nat.check(nat.lib.fcr_plan_shards(1, m, world, rank, C.byref(sh)), "fcr_plan_shards")
        assert sh.needs_reduce == 1 and sh.head_hi - sh.head_lo == 1
        rows_seen += sum(sh.row_hi[r] - sh.row_lo[r] for r in range(sh.n_ranges))
        sh.world = 1  # this test combines the partial vectors itself
        ws = torch.empty(nat.lib.fcr_sharded_workspace_bytes(C.byref(prob), C.byref(sh)), dtype=torch.uint8, device=dev)
        acc = torch.empty(1, n, dtype=torch.float32, device=dev)
        part = torch.empty(1, n, dtype=torch.float32, device=dev)
        nat.check(nat.lib.fcr_colreduce_sharded(C.byref(prob), C.byref(sh), 1, qd.data_ptr(), kd.data_ptr(), acc.data_ptr(),
                                                part.data_ptr(), nat.FCR_F32, ws.data_ptr(), ws.numel(), None, stream),
                  "fcr_colreduce_sharded")
        total = torch.maximum(total, part) if reduction == "max" else total + part
    assert rows_seen == m
    assert_parity(total[None], oracle_colreduce(q, k, reduction, causal), reduction)
