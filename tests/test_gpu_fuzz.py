"""Seeded random shapes against the oracle: every kernel family (general, few-tile items, 512-byte rows,
key streaming), ragged sizes, M > N, both masks, all reductions and dtypes, more work items than CTAs."""
import os

import pytest
import torch

from conftest import assert_parity
from oracle import oracle_colreduce

pytestmark = pytest.mark.gpu


def _case(seed: int):
    g = torch.Generator().manual_seed(1000 + seed)

    def pick(values):
        return values[int(torch.randint(len(values), (1,), generator=g))]

    family = seed % 4
    if family == 0:    # general kernels, several blocks per head
        m, n = pick([129, 300, 513, 777, 1100]), pick([100, 257, 640, 1500, 2304])
        heads = pick([1, 3, 40])
        d = pick([16, 40, 64, 72, 128])
    elif family == 1:  # decode shapes (one query tile, at least eight key tiles)
        m, n = pick([1, 5, 32, 33, 96, 128]), pick([1024, 1027, 2500, 4096, 6000])
        heads = pick([1, 7, 150])
        d = pick([32, 64, 80, 128])
    elif family == 2:  # 512-byte operand rows
        m, n = pick([64, 200, 400]), pick([128, 300, 1200])
        heads = pick([1, 5])
        d = pick([136, 192, 256])
    else:              # tiny and degenerate
        m, n = pick([1, 2, 127, 128]), pick([1, 3, 128, 129, 900])
        heads = pick([1, 2, 33])
        d = pick([8, 24, 128])
    dtype = pick([torch.float16, torch.float16, torch.bfloat16, torch.float32])
    if dtype == torch.float32 and d > 128:
        dtype = torch.float16
    b = 2 if heads % 2 == 0 and heads > 1 else 1
    h = heads // b
    scale = pick([None, None, 0.05, -0.2])
    q = torch.randn(b, h, m, d, generator=g)
    k = torch.randn(b, h, n, d, generator=g)
    if dtype == torch.float32:  # values exactly representable as TF32
        q = (q.view(torch.int32) & ~0x1FFF).view(torch.float32)
        k = (k.view(torch.int32) & ~0x1FFF).view(torch.float32)
    return q.to(dtype), k.to(dtype), scale


# FCR_FUZZ_CASES widens the sweep for a one-off soak run
@pytest.mark.parametrize("seed", range(int(os.environ.get("FCR_FUZZ_CASES", "128"))))
def test_random_case(seed):
    from flash_colreduce_b200 import flash_colreduce

    dev = torch.device("cuda", 0)
    q, k, scale = _case(seed)
    extra = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.float32: 0.0}[q.dtype]
    for red in ("sum", "mean", "max"):
        for causal in (False, True):
            got = flash_colreduce(q.to(dev), k.to(dev), red, is_causal=causal, scale=scale)
            assert got.dtype == q.dtype and got.shape == (q.shape[0], q.shape[1], k.shape[2])
            want = oracle_colreduce(q, k, red, causal, scale=scale)
            assert_parity(got.float().cpu(), want, red, extra_rtol=extra)
